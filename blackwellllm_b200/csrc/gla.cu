// Gated linear attention: a recurrent mixer with a matrix state per head and a decay per key channel.
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        S: [dk, dv] per head, float32, one per request
//   o_t = S_t^T q_t                            q scaled by q_scale
//   a_t = sigmoid(z_t) ^ (1 / tau) = exp(log_sigmoid(z_t) / tau)
//
// Everything but the projections that make q, k, v, z is float32 here: the decay and its logarithm,
// the state, the products that enter and leave it, and the norm of the head's output.
//
// gla_scan_kernel walks the tokens of one request's segment in order (a single decoded token and a
// portion of a prompt are the same case), from the state the steps before left in the request's slot,
// and leaves the new state there.  A block owns (request, head, COLS value columns); a column's dk state
// rows are spread over ROWSPLIT neighbouring lanes and live in registers.  The order of all sums
// depends on dk alone, never on how the tokens were cut into steps or on the batch.
//
// gla_gate_kernel: per token and head, o / rms(o) * gain * silu(g) -> the output projection's operand.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int ROWSPLIT = 8;     // lanes that share one value column
constexpr int COLS = 32;        // value columns of a block
constexpr int THREADS = ROWSPLIT * COLS;
constexpr int TOK_CHUNK = 8;    // tokens staged in shared memory at a time

struct ScanParams {
    const float* qkv;      // [T, ld]: q at q_off, k at k_off, v at v_off (head-major within each)
    const float* z;        // [T, heads * dk]: decay logits (bias added)
    const int* cu_q;       // [R + 1]
    const int* state_slot; // [R]
    float* state;          // [slots, heads, dk, dv]
    float* o;              // [T, heads * dv]
    long long ld;
    int q_off, k_off, v_off;
    int heads, dk, dv;
    float q_scale, inv_tau;
};

__device__ __forceinline__ float log_sigmoid(float z) {
    // log(1 / (1 + exp(-z))) without overflow on either side
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

template <int RPT>   // state rows per thread: dk <= ROWSPLIT * RPT
__global__ void __launch_bounds__(THREADS)
gla_scan_kernel(ScanParams p) {
    BW_PDL_TRIGGER();
    extern __shared__ float sm[];
    float* qs = sm;                          // [TOK_CHUNK][dk]
    float* ks = qs + TOK_CHUNK * p.dk;
    float* as = ks + TOK_CHUNK * p.dk;
    float* vs = as + TOK_CHUNK * p.dk;       // [TOK_CHUNK][COLS]
    const int r = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int rs = threadIdx.x % ROWSPLIT, col = threadIdx.x / ROWSPLIT;
    const int c = c0 + col;
    const bool col_ok = c < p.dv;
    const int t0 = p.cu_q[r], t1 = p.cu_q[r + 1];
    float* S = p.state + (((size_t)p.state_slot[r] * p.heads + h) * p.dk) * p.dv;
    BW_PDL_WAIT();
    float s[RPT];
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
        const int i = rs + ROWSPLIT * j;
        s[j] = (col_ok && i < p.dk) ? S[(size_t)i * p.dv + c] : 0.f;
    }
    for (int tb = t0; tb < t1; tb += TOK_CHUNK) {
        const int n = min(TOK_CHUNK, t1 - tb);
        __syncthreads();
        for (int idx = threadIdx.x; idx < n * p.dk; idx += THREADS) {
            const int tt = idx / p.dk, i = idx - tt * p.dk;
            const float* row = p.qkv + (size_t)(tb + tt) * p.ld;
            qs[idx] = row[p.q_off + h * p.dk + i] * p.q_scale;
            ks[idx] = row[p.k_off + h * p.dk + i];
            as[idx] = expf(log_sigmoid(p.z[(size_t)(tb + tt) * p.heads * p.dk + h * p.dk + i]) * p.inv_tau);
        }
        for (int idx = threadIdx.x; idx < n * COLS; idx += THREADS) {
            const int tt = idx / COLS, cc = idx - tt * COLS;
            vs[idx] = (c0 + cc < p.dv) ? p.qkv[(size_t)(tb + tt) * p.ld + p.v_off + h * p.dv + c0 + cc] : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float v = vs[tt * COLS + col];
            const float* q = qs + tt * p.dk;
            const float* k = ks + tt * p.dk;
            const float* a = as + tt * p.dk;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < RPT; ++j) {
                const int i = rs + ROWSPLIT * j;
                if (i < p.dk) {
                    s[j] = fmaf(a[i], s[j], k[i] * v);
                    acc = fmaf(s[j], q[i], acc);
                }
            }
#pragma unroll
            for (int o = ROWSPLIT / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (rs == 0 && col_ok) p.o[(size_t)(tb + tt) * p.heads * p.dv + h * p.dv + c] = acc;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
            const int i = rs + ROWSPLIT * j;
            if (i < p.dk) S[(size_t)i * p.dv + c] = s[j];
        }
    }
}

// one warp per (token, head): o / sqrt(mean(o^2) + eps) * gain[c] * silu(g[c])
template <typename OT>
__global__ void __launch_bounds__(128)
gla_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, long long g_ld, int g_off,
                const float* __restrict__ gain, OT* __restrict__ out, int T, int heads, int dv, float eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= T * heads) return;
    const int t = item / heads, h = item - t * heads;
    const float* orow = o + (size_t)t * heads * dv + (size_t)h * dv;
    const float* grow = g + (size_t)t * g_ld + g_off + (size_t)h * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = orow[c]; ss = fmaf(v, v, ss); }
    ss = bw::warp_sum(ss);
    const float r = rsqrtf(ss / (float)dv + eps);
    OT* dst = out + (size_t)t * heads * dv + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) {
        const float gv = grow[c];
        const float sg = gv / (1.f + expf(-gv));
        dst[c] = bw::from_f32<OT>(orow[c] * r * gain[c] * sg);
    }
}

}  // namespace

BW_EXPORT int bw_gla_scan(const float* qkv, long long ld, int q_off, int k_off, int v_off, const float* z,
                          const int* cu_q, const int* state_slot, float* state, float* o, int R, int heads, int dk,
                          int dv, float q_scale, float tau, void* stream) {
    if (R <= 0) return 0;
    if (heads <= 0 || dk <= 0 || dv <= 0 || !(tau > 0.f)) return BW_ERR_BAD_ARG;
    if (dk > ROWSPLIT * 32) return BW_ERR_UNSUPPORTED;
    ScanParams p;
    p.qkv = qkv; p.z = z; p.cu_q = cu_q; p.state_slot = state_slot; p.state = state; p.o = o; p.ld = ld;
    p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.heads = heads; p.dk = dk; p.dv = dv;
    p.q_scale = q_scale; p.inv_tau = 1.f / tau;
    const dim3 grid(R, heads, (dv + COLS - 1) / COLS);
    const size_t smem = (size_t)(3 * TOK_CHUNK * dk + TOK_CHUNK * COLS) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dk <= ROWSPLIT * 8) bw::launch((gla_scan_kernel<8>), grid, dim3(THREADS), smem, s, p);
    else if (dk <= ROWSPLIT * 16) bw::launch((gla_scan_kernel<16>), grid, dim3(THREADS), smem, s, p);
    else bw::launch((gla_scan_kernel<32>), grid, dim3(THREADS), smem, s, p);
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_gla_gate(const float* o, const float* g, long long g_ld, int g_off, const float* gain, void* out,
                          int out_type, int T, int heads, int dv, float eps, void* stream) {
    if (T <= 0) return 0;
    if (heads <= 0 || dv <= 0) return BW_ERR_BAD_ARG;
    const int items = T * heads;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32)
        bw::launch((gla_gate_kernel<float>), dim3((items + 3) / 4), dim3(128), 0, s, o, g, g_ld, g_off, gain, (float*)out, T, heads, dv, eps);
    else if (out_type == BW_BF16)
        bw::launch((gla_gate_kernel<bf16>), dim3((items + 3) / 4), dim3(128), 0, s, o, g, g_ld, g_off, gain, (bf16*)out, T, heads, dv, eps);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}
