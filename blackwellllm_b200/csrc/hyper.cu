// Hyper-connections: a layer's residual stream kept as S copies ("streams") x_1 .. x_S per token.  A sublayer
// reads a weighted sum of them and writes back through a mixing matrix:
//
//     u    = sum_s in[s] x_s                        what the sublayer's norm reads
//     x_t' = sum_s mix[s, t] x_s + out[t] y          all copies at once from the old ones; y = sublayer(norm(u))
//
// One kernel does the write of one sublayer and the read (with its RMS norm) of the next, since both walk
// the same rows: streams [T, S, H] float32 are read once, updated in place, the next sublayer's u stays in
// shared memory for its norm.  Every part is optional:
//   y == null        nothing is written back first (the first read of a model)
//   in == null       no read follows (the stream is only brought up to date)
//   gain == null     the read is written as float32 without a norm (the plain sum of the copies, with in = ones)
//   rows != null     only these rows are processed and the streams are left as they are (the last read of a
//                    model happens on the rows whose logits are wanted; the copies are not needed again)
// The norm is x / sqrt(mean(x^2) + eps) * gain with a float32 gain.  All arithmetic float32; one block per row.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int MAX_STREAMS = 8;

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
    *reinterpret_cast<uint2*>(p) = make_uint2(bw::pack_bf16x2(a, b), bw::pack_bf16x2(c, d));
}

// The same with four channels a thread and 16-byte accesses (H a multiple of 4, every pointer 16-byte aligned).
template <typename OT, int S>
__global__ void __launch_bounds__(256)
hc_step_vec4_kernel(float* __restrict__ streams, const float* __restrict__ y, const float* __restrict__ mix,
                    const float* __restrict__ out_w, const float* __restrict__ in_w, const float* __restrict__ gain,
                    const int* __restrict__ rows, OT* __restrict__ out, int H, float eps, int write_back,
               const float* __restrict__ planes, int n_planes, size_t plane_stride, int y_valid) {
    BW_PDL_TRIGGER();
    extern __shared__ __align__(16) float urow[];
    __shared__ float scratch[32];
    __shared__ float s_mix[S * S], s_out[S], s_in[S];
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = y ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
    if (threadIdx.x < S) { s_out[threadIdx.x] = y ? out_w[threadIdx.x] : 0.f; s_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 0.f; }
    __syncthreads();
    BW_PDL_WAIT();
    const int t = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xs = streams + (size_t)t * S * H;
    const float* yr = y ? y + (size_t)t * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        float4 old[S], now[S];
#pragma unroll
        for (int s = 0; s < S; ++s) old[s] = *reinterpret_cast<const float4*>(xs + (size_t)s * H + c);
        if (yr) {
            float4 yv = y_valid ? *reinterpret_cast<const float4*>(yr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = 0; p < n_planes; ++p) {   // a product's open sum: its planes are added here, in plane order
                const float4 pv = *reinterpret_cast<const float4*>(planes + (size_t)p * plane_stride + (size_t)t * H + c);
                yv.x += pv.x; yv.y += pv.y; yv.z += pv.z; yv.w += pv.w;
            }
#pragma unroll
            for (int r = 0; r < S; ++r) {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < S; ++s) {
                    const float m = s_mix[s * S + r];
                    a.x = fmaf(m, old[s].x, a.x); a.y = fmaf(m, old[s].y, a.y); a.z = fmaf(m, old[s].z, a.z); a.w = fmaf(m, old[s].w, a.w);
                }
                const float o = s_out[r];
                now[r] = make_float4(fmaf(o, yv.x, a.x), fmaf(o, yv.y, a.y), fmaf(o, yv.z, a.z), fmaf(o, yv.w, a.w));
            }
            if (write_back) {
#pragma unroll
                for (int r = 0; r < S; ++r) *reinterpret_cast<float4*>(xs + (size_t)r * H + c) = now[r];
            }
        } else {
#pragma unroll
            for (int r = 0; r < S; ++r) now[r] = old[r];
        }
        if (in_w) {
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const float w = s_in[s];
                u.x = fmaf(w, now[s].x, u.x); u.y = fmaf(w, now[s].y, u.y); u.z = fmaf(w, now[s].z, u.z); u.w = fmaf(w, now[s].w, u.w);
            }
            *reinterpret_cast<float4*>(urow + c) = u;
            ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
        }
    }
    if (!in_w) return;
    OT* o = out + (size_t)blockIdx.x * H;
    float r = 1.f;
    if (gain) r = rsqrtf(bw::block_sum(ss, scratch) / (float)H + eps);
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {   // each thread reads back what it wrote
        const float4 u = *reinterpret_cast<const float4*>(urow + c);
        const float4 g = gain ? *reinterpret_cast<const float4*>(gain + c) : make_float4(1.f, 1.f, 1.f, 1.f);
        store4(o + c, u.x * r * g.x, u.y * r * g.y, u.z * r * g.z, u.w * r * g.w);
    }
}

template <typename OT, int S>
__global__ void __launch_bounds__(256)
hc_step_kernel(float* __restrict__ streams, const float* __restrict__ y, const float* __restrict__ mix,
               const float* __restrict__ out_w, const float* __restrict__ in_w, const float* __restrict__ gain,
               const int* __restrict__ rows, OT* __restrict__ out, int H, float eps, int write_back,
               const float* __restrict__ planes, int n_planes, size_t plane_stride, int y_valid) {
    BW_PDL_TRIGGER();
    extern __shared__ __align__(16) float urow[];   // [H]: the next sublayer's input before its norm
    __shared__ float scratch[32];
    __shared__ float s_mix[S * S], s_out[S], s_in[S];
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = y ? mix[threadIdx.x] : ((threadIdx.x / S == threadIdx.x % S) ? 1.f : 0.f);
    if (threadIdx.x < S) { s_out[threadIdx.x] = y ? out_w[threadIdx.x] : 0.f; s_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 0.f; }
    __syncthreads();
    BW_PDL_WAIT();
    const int t = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xs = streams + (size_t)t * S * H;
    const float* yr = y ? y + (size_t)t * H : nullptr;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float old[S], now[S];
#pragma unroll
        for (int s = 0; s < S; ++s) old[s] = xs[(size_t)s * H + c];
        if (yr) {
            float yv = y_valid ? yr[c] : 0.f;
            for (int p = 0; p < n_planes; ++p) yv += planes[(size_t)p * plane_stride + (size_t)t * H + c];
#pragma unroll
            for (int r = 0; r < S; ++r) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < S; ++s) a = fmaf(s_mix[s * S + r], old[s], a);   // mix is indexed [from, to]
                now[r] = fmaf(s_out[r], yv, a);
            }
            if (write_back) {
#pragma unroll
                for (int r = 0; r < S; ++r) xs[(size_t)r * H + c] = now[r];
            }
        } else {
#pragma unroll
            for (int r = 0; r < S; ++r) now[r] = old[r];
        }
        if (in_w) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < S; ++s) u = fmaf(s_in[s], now[s], u);
            urow[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!in_w) return;
    OT* o = out + (size_t)blockIdx.x * H;
    if (!gain) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = bw::from_f32<OT>(urow[c]);   // each thread reads back what it wrote
        return;
    }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = bw::from_f32<OT>(urow[c] * r * gain[c]);
}

template <typename OT, int S>
int launch_hc(float* streams, const float* y, const float* mix, const float* out_w, const float* in_w, const float* gain,
              const int* rows, void* out, int n, int H, float eps, int write_back, const float* planes, int n_planes,
              size_t plane_stride, int y_valid, cudaStream_t s) {
    static bool raised[bw::MAX_DEVICES] = {}, raised4[bw::MAX_DEVICES] = {};
    const size_t smem = (size_t)H * sizeof(float);
    const bool vec = (H & 3) == 0 && (plane_stride & 3) == 0 &&
                     (((uintptr_t)streams | (uintptr_t)y | (uintptr_t)gain | (uintptr_t)out | (uintptr_t)planes) & 15) == 0;
    if (vec) {
        if (smem > 48 * 1024 && bw::allow_dynamic_smem(hc_step_vec4_kernel<OT, S>, 200 * 1024, raised4) != cudaSuccess) return BW_ERR_DRIVER;
        const int threads = H >= 1024 ? 256 : 128;
        bw::launch((hc_step_vec4_kernel<OT, S>), dim3(n), dim3(threads), smem, s, streams, y, mix, out_w, in_w, gain, rows, (OT*)out, H, eps,
                   write_back, planes, n_planes, plane_stride, y_valid);
        BW_LAUNCH_CHECK();
        return 0;
    }
    if (smem > 48 * 1024 && bw::allow_dynamic_smem(hc_step_kernel<OT, S>, 200 * 1024, raised) != cudaSuccess) return BW_ERR_DRIVER;
    bw::launch((hc_step_kernel<OT, S>), dim3(n), dim3(256), smem, s, streams, y, mix, out_w, in_w, gain, rows, (OT*)out, H, eps, write_back, planes, n_planes,
               plane_stride, y_valid);
    BW_LAUNCH_CHECK();
    return 0;
}

template <typename OT>
int dispatch_streams(int S, float* streams, const float* y, const float* mix, const float* out_w, const float* in_w,
                     const float* gain, const int* rows, void* out, int n, int H, float eps, int write_back,
                     const float* planes, int n_planes, size_t plane_stride, int y_valid, cudaStream_t s) {
    switch (S) {
#define BW_HC(N) case N: return launch_hc<OT, N>(streams, y, mix, out_w, in_w, gain, rows, out, n, H, eps, write_back, planes, n_planes, \
                                                 plane_stride, y_valid, s);
        BW_HC(1) BW_HC(2) BW_HC(3) BW_HC(4) BW_HC(5) BW_HC(6) BW_HC(7) BW_HC(8)
#undef BW_HC
    }
    return BW_ERR_UNSUPPORTED;
}

}  // namespace

// streams float32 [T, S, H] (updated in place when y is given and write_back != 0); y float32 [T, H] or null;
// mix float32 [S, S] indexed [from, to], out_w float32 [S] (both needed with y); in_w float32 [S] or null;
// gain float32 [H] or null; rows int32 [n] or null (then n = T rows, all); out [n, H] of out_type (float32
// when there is no gain).  S up to 8; H * 4 bytes up to 200 KB.
// planes (with y): n_planes float32 planes [T, H], plane_stride floats apart, that are added to y's rows in plane order as
// they are read (a matrix product's K splits left unsummed); y_valid == 0: y's own values are not read, the planes are all of it.
BW_EXPORT int bw_hc_step(float* streams, const float* y, const float* mix, const float* out_w, const float* in_w,
                         const float* gain, const int* rows, void* out, int out_type, int n, int S, int H, float eps,
                         int write_back, const float* planes, int n_planes, long long plane_stride, int y_valid, void* stream) {
    if (n <= 0) return 0;
    if (!planes) n_planes = 0;
    if (n_planes < 0 || plane_stride < 0 || (!y_valid && n_planes == 0 && y)) return BW_ERR_BAD_ARG;
    if (!streams || H <= 0 || (size_t)H * sizeof(float) > 200 * 1024 || (y && (!mix || !out_w)) || (in_w && !out) ||
        (!gain && in_w && out_type != BW_F32) || (rows && write_back))
        return BW_ERR_BAD_ARG;
    if (S < 1 || S > MAX_STREAMS) return BW_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32) return dispatch_streams<float>(S, streams, y, mix, out_w, in_w, gain, rows, out, n, H, eps, write_back, planes,
                                                           n_planes, (size_t)plane_stride, y_valid, s);
    if (out_type == BW_BF16) return dispatch_streams<bf16>(S, streams, y, mix, out_w, in_w, gain, rows, out, n, H, eps, write_back, planes,
                                                           n_planes, (size_t)plane_stride, y_valid, s);
    return BW_ERR_BAD_ARG;
}
