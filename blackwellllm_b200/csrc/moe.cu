// Routed feed-forward (mixture of experts): router scores, the choice of experts, the regrouping of
// the step's tokens by expert, the experts' two matrix products over the regrouped rows, and the sum of
// each token's expert outputs.  Nothing here goes through the host: the number of rows an expert gets is
// known on the device only, so the kernels are launched for the worst case and idle tiles return at once
// (a decode step stays capturable in a CUDA graph).
//
//   moe_route    one warp per token: score = sigmoid(logit) (or softmax), the `top` largest scores
//                (lowest index on ties), optionally renormalised to sum 1; float32 throughout.  With a bias
//                per router output the CHOICE goes by score + bias while the weights stay the scores.
//                The router may have more outputs than there are experts: outputs from `E` (the experts
//                that have weights) up to `E_total` stand for experts that return their input; their rows
//                take no part in the regrouping and the products, and moe_combine adds weight * x for them
//   moe_plan     one block: rows per expert, each expert's stretch padded to whole tiles (64 rows here, 128 in moe_tc.cu),
//                the place of every (token, choice) row, and the expert of every tile
//   moe_scatter  the regrouped operand: row (token, choice) = weight * x[token] (input scaling) or x[token]
//   moe_gemm     C[row, :] = A[row, :] W[expert of row]^T, optionally as silu(A Wg^T) * (A Wu^T);
//                float32 sums on the CUDA cores from float32 or bfloat16 operands (the true 32-bit path, and
//                bfloat16 sizes that the tcgen05 kernel of moe_tc.cu does not take)
//   moe_combine  out[token] = sum over choices (in order) of (weight *) C[row of (token, choice)], written,
//                added to a stream, or normalised (RMS, gain) and then added to a stream
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int TILE_M = 64;   // rows of a tile of regrouped tokens; also the padding of an expert's stretch
constexpr int BN = 64, BK = 16;

// dst[c] = src[c] * w over a row of H elements, thread `me` of `n`; 16-byte accesses when the row allows
__device__ __forceinline__ void scale_row(const float* __restrict__ src, float* __restrict__ dst, int H, float w, int me, int n) {
    if ((H & 3) == 0) {
        for (int c = me * 4; c < H; c += n * 4) {
            float4 v = *reinterpret_cast<const float4*>(src + c);
            v.x *= w; v.y *= w; v.z *= w; v.w *= w;
            *reinterpret_cast<float4*>(dst + c) = v;
        }
    } else {
        for (int c = me; c < H; c += n) dst[c] = src[c] * w;
    }
}
__device__ __forceinline__ void scale_row(const bf16* __restrict__ src, bf16* __restrict__ dst, int H, float w, int me, int n) {
    if ((H & 7) == 0) {
        for (int c = me * 8; c < H; c += n * 8) {
            uint4 raw = *reinterpret_cast<const uint4*>(src + c);
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(h[k]); h[k] = __floats2bfloat162_rn(f.x * w, f.y * w); }
            *reinterpret_cast<uint4*>(dst + c) = raw;
        }
    } else {
        for (int c = me; c < H; c += n) dst[c] = __float2bfloat16_rn(__bfloat162float(src[c]) * w);
    }
}

// ---------------------------------------------------------------- routing
// E: the router's outputs; bias: float32 [E] added to the scores for the choice only, or null; renorm_eps: added to
// the sum of the chosen scores before they are divided by it
__device__ __forceinline__ void route_token(const float* __restrict__ logits, int t, int lane, int E, int top, int softmax,
                                            int renorm, const float* __restrict__ bias, float renorm_eps,
                                            int* __restrict__ sel, float* __restrict__ wt) {
    const float* z = logits + (size_t)t * E;
    float zmax = -INFINITY, zsum = 0.f;
    if (softmax) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = bw::warp_max(zmax);
        for (int e = lane; e < E; e += 32) zsum += expf(z[e] - zmax);
        zsum = bw::warp_sum(zsum);
    }
    float total = 0.f;
    int last = -1; float last_s = INFINITY;   // choices are taken in order of (choice score descending, index ascending)
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, best_w = 0.f; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float w = softmax ? expf(z[e] - zmax) / zsum : 1.f / (1.f + expf(-z[e]));
            const float s = bias ? w + bias[e] : w;
            const bool after = (s < last_s) || (s == last_s && e > last);   // not chosen yet
            if (after && (s > best || (s == best && e < bi))) { best = s; best_w = w; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const float ow = __shfl_xor_sync(0xffffffffu, best_w, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; best_w = ow; bi = oi; }
        }
        last = bi; last_s = best; total += best_w;
        if (lane == 0) { sel[(size_t)t * top + k] = bi; wt[(size_t)t * top + k] = best_w; }
    }
    total += renorm_eps;
    if (renorm && lane == 0 && total > 0.f)
        for (int k = 0; k < top; ++k) wt[(size_t)t * top + k] /= total;
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int T, int E, int top, int softmax, int renorm,
                 const float* __restrict__ bias, float renorm_eps, int* __restrict__ sel, float* __restrict__ wt) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    route_token(logits, t, lane, E, top, softmax, renorm, bias, renorm_eps, sel, wt);
}

// ---------------------------------------------------------------- plan
// pos_of[n] for the n = T * top rows (token-major; -1 for a row whose choice is no expert with weights, i.e. >= E);
// tile_expert[max_tiles] (-1: idle tile).
__device__ __forceinline__ void plan_block(const int* __restrict__ sel, int n, int E, int tile_rows, int max_tiles,
                                           int* __restrict__ pos_of, int* __restrict__ tile_expert, int* sh) {
    int* count = sh;          // [E]
    int* start = sh + E;      // [E + 1], in rows
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = sel[i];
        pos_of[i] = (e >= 0 && e < E) ? atomicAdd(&count[e], 1) : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) { start[e] = at; at += (count[e] + tile_rows - 1) / tile_rows * tile_rows; }
        start[E] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = sel[i];
        if (e >= 0 && e < E) pos_of[i] += start[e];
    }
    for (int tile = threadIdx.x; tile < max_tiles; tile += blockDim.x) {
        const int row = tile * tile_rows;
        int e = -1;
        if (row < start[E]) {
            int lo = 0, hi = E - 1;            // the last expert whose stretch starts at or before row
            while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (start[mid] <= row) lo = mid; else hi = mid - 1; }
            e = lo;
            if (row >= start[e] + count[e]) e = -1;   // wholly inside an expert's padding (cannot happen: the padding is less than a tile)
        }
        tile_expert[tile] = e;
    }
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ sel, int n, int E, int tile_rows, int max_tiles, int* __restrict__ pos_of,
                int* __restrict__ tile_expert) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    extern __shared__ int sh[];
    plan_block(sel, n, E, tile_rows, max_tiles, pos_of, tile_expert, sh);
}

// The three steps above as one block, for steps of few tokens (a decode step): choice, plan and regrouped operand
// without two more launches.  The block's own writes to sel, wt and pos_of are read back after a barrier.
template <typename XT>
__global__ void __launch_bounds__(1024)
moe_route_plan_scatter_kernel(const float* __restrict__ logits, int T, int E, int E_total, int top, int softmax, int renorm,
                              const float* __restrict__ bias, float renorm_eps,
                              int* __restrict__ sel, float* __restrict__ wt, int tile_rows, int max_tiles,
                              int* __restrict__ pos_of, int* __restrict__ tile_expert, const XT* __restrict__ x,
                              XT* __restrict__ xs, int H, int scale_input) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    extern __shared__ int sh[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < T; t += 32) route_token(logits, t, lane, E_total, top, softmax, renorm, bias, renorm_eps, sel, wt);
    __syncthreads();
    plan_block(sel, T * top, E, tile_rows, max_tiles, pos_of, tile_expert, sh);
    __syncthreads();
    for (int i = warp; i < T * top; i += 32) {
        if (pos_of[i] < 0) continue;
        const float w = scale_input ? wt[i] : 1.f;
        const XT* src = x + (size_t)(i / top) * H;
        XT* dst = xs + (size_t)pos_of[i] * H;
        scale_row(src, dst, H, w, lane, 32);
    }
}

// ---------------------------------------------------------------- scatter
template <typename XT>
__global__ void __launch_bounds__(256)
moe_scatter_kernel(const XT* __restrict__ x, const int* __restrict__ pos_of, const float* __restrict__ wt,
                   XT* __restrict__ xs, int H, int top, int scale_input) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int i = blockIdx.x;                 // (token, choice)
    if (pos_of[i] < 0) return;                // an expert without weights: nothing to regroup
    const int t = i / top;
    const float w = scale_input ? wt[i] : 1.f;
    const XT* src = x + (size_t)t * H;
    XT* dst = xs + (size_t)pos_of[i] * H;
    scale_row(src, dst, H, w, threadIdx.x, blockDim.x);
}

// ---------------------------------------------------------------- grouped product
// A [rows, K], W [E, N, K] (and W2 the same for GATED), C [rows, N].  grid (max_tiles, ceil(N / BN)).
template <typename AT, typename CT, bool GATED>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const AT* __restrict__ A, const AT* __restrict__ W, const AT* __restrict__ W2,
                const int* __restrict__ tile_expert, CT* __restrict__ C, int N, int K, int act, float limit, float alpha) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    __shared__ float As[BK][TILE_M + 4];
    __shared__ float Bs[BK][BN + 4];
    __shared__ float B2s[GATED ? BK : 1][BN + 4];
    const int row0 = blockIdx.x * TILE_M, n0 = blockIdx.y * BN;
    const AT* Wb = W + (size_t)e * N * K;
    const AT* W2b = GATED ? W2 + (size_t)e * N * K : nullptr;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {}, acc2[GATED ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = threadIdx.x; idx < TILE_M * BK; idx += 256) {
            const int m = idx / BK, kk = idx % BK;
            As[kk][m] = (k0 + kk < K) ? bw::to_f32(A[(size_t)(row0 + m) * K + k0 + kk]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
            const int nn = idx / BK, kk = idx % BK;
            const bool ok = n0 + nn < N && k0 + kk < K;
            Bs[kk][nn] = ok ? bw::to_f32(Wb[(size_t)(n0 + nn) * K + k0 + kk]) : 0.f;
            if constexpr (GATED) B2s[kk][nn] = ok ? bw::to_f32(W2b[(size_t)(n0 + nn) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; if constexpr (GATED) b2[i] = B2s[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if constexpr (GATED) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if constexpr (GATED) v = bw::glu(act, v, acc2[i][j], limit, alpha);
            C[(size_t)(row0 + ty * 4 + i) * N + n] = bw::from_f32<CT>(v);
        }
}

// ---------------------------------------------------------------- combine
// mode 0: out = sum; 1: out += sum; 2: out += sum / rms(sum) * gain.  One block per token.  A choice without a
// place (pos_of < 0: an expert that returns its input) contributes the token's own row of x.
template <typename XT>
__device__ __forceinline__ float4 row4(const XT* p);
template <> __device__ __forceinline__ float4 row4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 row4<bf16>(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename XT>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ pos_of, const float* __restrict__ wt,
                   int top, int scale_output, float* __restrict__ out, int H, int mode,
                   const float* __restrict__ gain, float eps, const XT* __restrict__ x) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    extern __shared__ __align__(16) float row[];    // [H]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    float ss = 0.f;
    const bool vec = (H & 3) == 0;
    if (vec) {
        for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const float w = scale_output ? wt[(size_t)t * top + k] : 1.f;
                const int at = pos_of[(size_t)t * top + k];
                const float4 a = at >= 0 ? *reinterpret_cast<const float4*>(y + (size_t)at * H + c)
                                         : (x ? row4<XT>(x + (size_t)t * H + c) : make_float4(0.f, 0.f, 0.f, 0.f));
                v.x = fmaf(w, a.x, v.x); v.y = fmaf(w, a.y, v.y); v.z = fmaf(w, a.z, v.z); v.w = fmaf(w, a.w, v.w);
            }
            *reinterpret_cast<float4*>(row + c) = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = 0.f;
            for (int k = 0; k < top; ++k) {
                const float w = scale_output ? wt[(size_t)t * top + k] : 1.f;
                const int at = pos_of[(size_t)t * top + k];
                v = fmaf(w, at >= 0 ? y[(size_t)at * H + c] : (x ? bw::to_f32(x[(size_t)t * H + c]) : 0.f), v);
            }
            row[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    float r = 1.f;
    if (mode == 2) r = rsqrtf(bw::block_sum(ss, scratch) / (float)H + eps);
    float* o = out + (size_t)t * H;
    if (vec) {
        for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {   // each thread reads back what it wrote
            const float4 v = *reinterpret_cast<const float4*>(row + c);
            float4 d = mode == 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(o + c);
            if (mode == 2) {
                const float4 g = *reinterpret_cast<const float4*>(gain + c);
                d.x += v.x * r * g.x; d.y += v.y * r * g.y; d.z += v.z * r * g.z; d.w += v.w * r * g.w;
            } else { d.x += v.x; d.y += v.y; d.z += v.z; d.w += v.w; }
            *reinterpret_cast<float4*>(o + c) = d;
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float v = row[c];
            if (mode == 0) o[c] = v;
            else if (mode == 1) o[c] += v;
            else o[c] += v * r * gain[c];
        }
    }
}

}  // namespace

BW_EXPORT int bw_moe_tile_rows() { return TILE_M; }

// E: the router's outputs (logits [T, E]); bias: float32 [E] or null; renorm_eps: see route_token
BW_EXPORT int bw_moe_route(const float* logits, int T, int E, int top, int softmax, int renorm, const float* bias,
                           float renorm_eps, int* sel, float* wt, void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E) return BW_ERR_BAD_ARG;
    bw::launch((moe_route_kernel), dim3((T + 3) / 4), dim3(128), 0, (cudaStream_t)stream, logits, T, E, top, softmax, renorm, bias,
               renorm_eps, sel, wt);
    BW_LAUNCH_CHECK();
    return 0;
}

// tile_rows: rows of a tile (what the product kernel that follows works on); an expert's stretch is padded to it
BW_EXPORT int bw_moe_plan(const int* sel, int n, int E, int tile_rows, int max_tiles, int* pos_of, int* tile_expert, void* stream) {
    if (n <= 0) return 0;
    if (E <= 0 || E > 4096 || tile_rows <= 0 || max_tiles < (n + tile_rows - 1) / tile_rows + E) return BW_ERR_BAD_ARG;
    bw::launch((moe_plan_kernel), dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int), (cudaStream_t)stream, sel, n, E, tile_rows,
               max_tiles, pos_of, tile_expert);
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_moe_scatter(const void* x, int type, const int* pos_of, const float* wt, void* xs, int n, int H, int top,
                             int scale_input, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (type == BW_F32) bw::launch((moe_scatter_kernel<float>), dim3(n), dim3(256), 0, s, (const float*)x, pos_of, wt, (float*)xs, H, top, scale_input);
    else if (type == BW_BF16) bw::launch((moe_scatter_kernel<bf16>), dim3(n), dim3(256), 0, s, (const bf16*)x, pos_of, wt, (bf16*)xs, H, top, scale_input);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// E: experts with weights; E_total >= E: the router's outputs (logits [T, E_total], bias [E_total] or null)
BW_EXPORT int bw_moe_route_plan_scatter(const float* logits, int T, int E, int E_total, int top, int softmax, int renorm,
                                        const float* bias, float renorm_eps, int* sel, float* wt,
                                        int tile_rows, int max_tiles, int* pos_of, int* tile_expert, const void* x, int type,
                                        void* xs, int H, int scale_input, void* stream) {
    if (T <= 0) return 0;
    const int n = T * top;
    if (E <= 0 || E > 4096 || E_total < E || top <= 0 || top > E_total || n > 1024 || tile_rows <= 0 ||
        max_tiles < (n + tile_rows - 1) / tile_rows + E)
        return BW_ERR_BAD_ARG;
    const size_t smem = (size_t)(2 * E + 1) * sizeof(int);
    cudaStream_t s = (cudaStream_t)stream;
#define BW_RPS(XT) bw::launch((moe_route_plan_scatter_kernel<XT>), dim3(1), dim3(1024), smem, s, logits, T, E, E_total, top, softmax, renorm, bias, renorm_eps, sel, wt, \
        tile_rows, max_tiles, pos_of, tile_expert, (const XT*)x, (XT*)xs, H, scale_input)
    if (type == BW_F32) BW_RPS(float);
    else if (type == BW_BF16) BW_RPS(bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_RPS
    BW_LAUNCH_CHECK();
    return 0;
}

// type: element type of A and the weights; c_type: of C.  w2 non-null: C = glu(A w^T, A w2^T) with the gated
// activation `act` of common.cuh (BW_ACT_SILU: silu(A w^T) * (A w2^T)) and its limit and alpha.
BW_EXPORT int bw_moe_gemm(const void* A, const void* w, const void* w2, int type, const int* tile_expert, void* C, int c_type,
                          int max_tiles, int N, int K, int act, float limit, float alpha, void* stream) {
    if (max_tiles <= 0) return 0;
    if (N <= 0 || K <= 0) return BW_ERR_BAD_ARG;
    const dim3 grid(max_tiles, (N + BN - 1) / BN);
    cudaStream_t s = (cudaStream_t)stream;
#define BW_MG(AT, CT, G) bw::launch((moe_gemm_kernel<AT, CT, G>), grid, dim3(256), 0, s, (const AT*)A, (const AT*)w, (const AT*)w2, tile_expert, (CT*)C, N, K, act, limit, alpha)
    if (type == BW_F32 && c_type == BW_F32) { if (w2) BW_MG(float, float, true); else BW_MG(float, float, false); }
    else if (type == BW_BF16 && c_type == BW_BF16) { if (w2) BW_MG(bf16, bf16, true); else BW_MG(bf16, bf16, false); }
    else if (type == BW_BF16 && c_type == BW_F32) { if (w2) BW_MG(bf16, float, true); else BW_MG(bf16, float, false); }
    else return BW_ERR_BAD_ARG;
#undef BW_MG
    BW_LAUNCH_CHECK();
    return 0;
}

// x (of x_type, [T, H]): the experts' input, read for choices without a place (experts that return their input);
// null where there are none.
BW_EXPORT int bw_moe_combine(const float* y, const int* pos_of, const float* wt, int top, int scale_output, float* out, int T,
                             int H, int mode, const float* gain, float eps, const void* x, int x_type, void* stream) {
    if (T <= 0) return 0;
    if (mode < 0 || mode > 2 || (mode == 2 && !gain) || (size_t)H * sizeof(float) > 200 * 1024) return BW_ERR_BAD_ARG;
    static bool raised[bw::MAX_DEVICES] = {}, raised_bf16[bw::MAX_DEVICES] = {};
    const size_t smem = (size_t)H * sizeof(float);
    if (x && x_type == BW_BF16) {
        if (smem > 48 * 1024 && bw::allow_dynamic_smem(moe_combine_kernel<bf16>, 200 * 1024, raised_bf16) != cudaSuccess) return BW_ERR_DRIVER;
        bw::launch((moe_combine_kernel<bf16>), dim3(T), dim3(256), smem, (cudaStream_t)stream, y, pos_of, wt, top, scale_output, out, H,
                   mode, gain, eps, (const bf16*)x);
    } else if (!x || x_type == BW_F32) {
        if (smem > 48 * 1024 && bw::allow_dynamic_smem(moe_combine_kernel<float>, 200 * 1024, raised) != cudaSuccess) return BW_ERR_DRIVER;
        bw::launch((moe_combine_kernel<float>), dim3(T), dim3(256), smem, (cudaStream_t)stream, y, pos_of, wt, top, scale_output, out, H,
                   mode, gain, eps, (const float*)x);
    } else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}
