// Query/key norm over the whole projection, rotary encoding and cache append in one kernel, for
// attention mixers whose q/k/v projection cannot carry the rotation in its own epilogue (the norm
// needs the whole row first) and whose heads may have a key size different from the value size.
//
// qkv: float32 [T, nh*dq + nkv*dq + nkv*dv] (queries, keys, values; biases already added).
//   * norm (optional, q_gain/k_gain non-null): all nh*dq query channels of a token are divided by their
//     common root mean square and multiplied by a gain per channel; the same for the nkv*dq key channels.
//   * rotation of the first rotary_dim channels of every q and k head with the step's cos/sin table
//     [T, rotary_dim] (cosines, then sines; any magnitude factor is already in the table).
//     interleaved != 0: channel 2i pairs with 2i + 1; else channel i pairs with i + rotary_dim / 2.
//   * q_out [T, nh, dpad], keys and values to the page of the token's position,
//     pages [num_pages, nkv, page_size, dpad]; channels from dq (dv) up to dpad are written as zeros, so
//     that an attention kernel built for one head size serves both.
// All arithmetic is float32; one block per token.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

template <typename OT>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                    const int* __restrict__ req_of_token, const int* __restrict__ block_table, int max_blocks,
                    const float* __restrict__ table, int rotary_dim, int interleaved,
                    const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                    OT* __restrict__ q_out, OT* __restrict__ k_pages, OT* __restrict__ v_pages,
                    int nh, int nkv, int dq, int dv, int dpad, int page_size, int num_pages) {
    BW_PDL_TRIGGER();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int nq = nh * dq, nk = nkv * dq, nv = nkv * dv;
    const int pos = positions[t];
    int page = -1;
    const int slot = pos % page_size;
    if (num_pages > 0) {
        page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
        if (page >= num_pages) page = -1;
    }
    BW_PDL_WAIT();
    const float* row = qkv + (size_t)t * (nq + nk + nv);
    float rq = 1.f, rk = 1.f;
    if (q_gain) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = row[c]; ss = fmaf(v, v, ss); }
        rq = rsqrtf(bw::block_sum(ss, scratch) / (float)nq + eps);
    }
    if (k_gain) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = row[nq + c]; ss = fmaf(v, v, ss); }
        rk = rsqrtf(bw::block_sum(ss, scratch) / (float)nk + eps);
    }
    const int half = rotary_dim >> 1;
    const float* tab = table + (size_t)t * rotary_dim;
    // queries and keys: heads 0..nh-1 are queries, nh..nh+nkv-1 keys
    const int n_qk = (nh + nkv) * dpad;
    for (int idx = threadIdx.x; idx < n_qk; idx += blockDim.x) {
        const int h = idx / dpad, c = idx - h * dpad;
        const bool is_q = h < nh;
        float o = 0.f;
        if (c < dq) {
            const float* src = is_q ? row + (size_t)h * dq : row + nq + (size_t)(h - nh) * dq;
            const float* gain = is_q ? (q_gain ? q_gain + (size_t)h * dq : nullptr)
                                     : (k_gain ? k_gain + (size_t)(h - nh) * dq : nullptr);
            const float r = is_q ? rq : rk;
            float x = src[c] * r;
            if (gain) x *= gain[c];
            o = x;
            if (c < rotary_dim) {
                int j, pc; bool first;
                if (interleaved) { j = c >> 1; pc = c ^ 1; first = !(c & 1); }
                else { first = c < half; j = first ? c : c - half; pc = first ? c + half : c - half; }
                float y = src[pc] * r;
                if (gain) y *= gain[pc];
                const float cs = tab[j], sn = tab[half + j];
                o = first ? x * cs - y * sn : x * cs + y * sn;
            }
        }
        if (is_q) q_out[((size_t)t * nh + h) * dpad + c] = bw::from_f32<OT>(o);
        else if (page >= 0) k_pages[(((size_t)page * nkv + (h - nh)) * page_size + slot) * dpad + c] = bw::from_f32<OT>(o);
    }
    if (page >= 0) {
        const float* vsrc = row + nq + nk;
        for (int idx = threadIdx.x; idx < nkv * dpad; idx += blockDim.x) {
            const int h = idx / dpad, c = idx - h * dpad;
            const float o = c < dv ? vsrc[(size_t)h * dv + c] : 0.f;
            v_pages[(((size_t)page * nkv + h) * page_size + slot) * dpad + c] = bw::from_f32<OT>(o);
        }
    }
}

}  // namespace

// out_type: element type of q_out and the pages.  num_pages <= 0: nothing is appended (a run that reads
// another run's cache).  q_gain / k_gain: float32 gains of the norm, or null for no norm.
BW_EXPORT int bw_qk_norm_rope_append(const float* qkv, const int* positions, const int* req_of_token,
                                     const int* block_table, int max_blocks, const float* table, int rotary_dim,
                                     int interleaved, const float* q_gain, const float* k_gain, float eps,
                                     void* q_out, void* k_pages, void* v_pages, int out_type, int T, int nh, int nkv,
                                     int dq, int dv, int dpad, int page_size, int num_pages, void* stream) {
    if (T <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > dq || (rotary_dim & 1) || dq <= 0 || dv <= 0 || dpad < dq || dpad < dv ||
        nh <= 0 || nkv <= 0 || page_size <= 0 || (rotary_dim > 0 && !table))
        return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
#define BW_QK(OT) bw::launch((qk_norm_rope_kernel<OT>), dim3(T), dim3(256), 0, s, qkv, positions, req_of_token, block_table, \
        max_blocks, table, rotary_dim, interleaved, q_gain, k_gain, eps, (OT*)q_out, (OT*)k_pages, (OT*)v_pages, nh, nkv, dq, dv, \
        dpad, page_size, num_pages)
    if (out_type == BW_F32) BW_QK(float);
    else if (out_type == BW_BF16) BW_QK(bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_QK
    BW_LAUNCH_CHECK();
    return 0;
}
