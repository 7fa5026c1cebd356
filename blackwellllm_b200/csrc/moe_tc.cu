// The experts' matrix products of a routed feed-forward on the tcgen05 tensor cores (bfloat16 in, float32
// sums in tensor memory).  The step's rows are regrouped by expert (moe.cu): tile t of 128 rows belongs to
// expert tile_expert[t] (-1: an idle tile, its CTAs return at once), and the experts' weights are one
// stacked tensor [E * N, K], so a tile's weight rows start at expert * N: one launch covers all experts,
// and nothing about the routing is known on the host.
//
// One CTA per (tile of 128 rows, 128 weight rows): warp 0 feeds a ring of TMA stages (128-byte swizzle),
// warp 1 owns the tensor memory and issues the MMAs (M = 128, N = 128, K = 16), warps 2..5 read the
// accumulator (TMEM lane quarter = warp % 4) and write the result: either plain (float32 or bfloat16), or,
// for a gate/up weight whose rows alternate in blocks of 16 (16 gate features, the same 16 up features),
// silu(gate) * up as bfloat16.  Three stages of 32 KB leave room for two CTAs on an SM.
// Every wait is bounded; a wait that gives up sets the status word and the roles fall through to the exit.
#include "tcgen05.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int BM = 128, BN = 128, BK = 64, UMMA_K = 16, STAGES = 3, THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 128;
constexpr uint32_t TMEM_COLS = 128;
constexpr uint32_t IDESC = bw::umma_idesc_bf16(BM, BN);
constexpr int GATE_BLOCK = 16;

__device__ int g_status = 0;

template <bool GATED, typename CT>
__global__ void __launch_bounds__(THREADS)
moe_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
              const int* __restrict__ tile_expert, CT* __restrict__ C, int N, int K, int act, float limit, float alpha) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);     // full[STAGES], empty[STAGES], done
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();               // the regrouped rows and the tiles' experts come from the kernels before
    const int e = tile_expert[blockIdx.y];
    if (e < 0) return;           // the whole CTA: nothing was allocated yet
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = bw::smem_u32(bars), empty0 = bw::smem_u32(bars + STAGES), done = bw::smem_u32(bars + 2 * STAGES);
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { bw::mbar_init(full0 + 8 * s, 1); bw::mbar_init(empty0 + 8 * s, 1); }
        bw::mbar_init(done, 1);
        bw::fence_barrier_init();
        bw::tma_prefetch_desc(&tmA);
        bw::tma_prefetch_desc(&tmB);
    }
    if (warp == 1) bw::tmem_alloc(bw::smem_u32(tmem_slot), TMEM_COLS);
    bw::tc_fence_before();
    __syncthreads();
    bw::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int row0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nkb = (K + BK - 1) / BK;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!bw::mbar_wait(empty0 + 8 * s, ph ^ 1, &g_status, 1)) break;
                const uint32_t dst = bw::smem_u32(smem + s * STAGE_BYTES);
                bw::mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                bw::tma_load_2d(dst, &tmA, full0 + 8 * s, i * BK, row0);
                bw::tma_load_2d(dst + A_BYTES, &tmB, full0 + 8 * s, i * BK, e * N + n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!bw::mbar_wait(full0 + 8 * s, ph, &g_status, 2)) { ok = false; break; }
                bw::tc_fence_after();
                const uint32_t a_addr = bw::smem_u32(smem + s * STAGE_BYTES);
                const uint64_t da = bw::umma_smem_desc_sw128(a_addr);
                const uint64_t db = bw::umma_smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)   // 32 bytes (2 units of 16) further along K inside the swizzle row
                    bw::umma_bf16(tmem_base, da + 2 * k, db + 2 * k, IDESC, (i | k) != 0);
                bw::umma_commit(empty0 + 8 * s);
            }
            if (ok) bw::umma_commit(done);
        }
    } else {
        const int quarter = warp & 3;
        if (bw::mbar_wait(done, 0, &g_status, 3)) {
            bw::tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const size_t row = (size_t)row0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                bw::tmem_ld_32x32(lane_addr + c0, v);
                bw::tmem_ld_wait();
                if constexpr (GATED) {
                    // weight rows n0 + c0 .. + 31: 16 gate rows, then the 16 up rows of the same features
                    const int F = N / 2;
                    const int f0 = (n0 + c0) / (2 * GATE_BLOCK) * GATE_BLOCK;
                    if (f0 < F) {
                        float y[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float g = __uint_as_float(v[i]), u = __uint_as_float(v[16 + i]);
                            if (act == BW_ACT_CLAMPED_SWISH) {   // g sigmoid(alpha g) (u + 1) on clamped g and u
                                g = fminf(g, limit);
                                u = fminf(fmaxf(u, -limit), limit) + 1.f;
                                y[i] = __fdividef(g, 1.f + __expf(-alpha * g)) * u;
                            } else {
                                y[i] = __fdividef(g, 1.f + __expf(-g)) * u;
                            }
                        }
                        bf16* dst = (bf16*)C + row * F + f0;
                        if ((F & 7) == 0) {
                            *reinterpret_cast<uint4*>(dst) = make_uint4(bw::pack_bf16x2(y[0], y[1]), bw::pack_bf16x2(y[2], y[3]),
                                                                        bw::pack_bf16x2(y[4], y[5]), bw::pack_bf16x2(y[6], y[7]));
                            *reinterpret_cast<uint4*>(dst + 8) = make_uint4(bw::pack_bf16x2(y[8], y[9]), bw::pack_bf16x2(y[10], y[11]),
                                                                            bw::pack_bf16x2(y[12], y[13]), bw::pack_bf16x2(y[14], y[15]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) dst[i] = __float2bfloat16_rn(y[i]);
                        }
                    }
                } else {
                    CT* dst = C + row * N + n0 + c0;
                    if (n0 + c0 + 32 <= N && (N & 3) == 0 && sizeof(CT) == 4) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c0 + j < N) dst[j] = bw::from_f32<CT>(__uint_as_float(v[j]));
                    }
                }
            }
        }
    }
    bw::tc_fence_before();
    __syncthreads();
    if (warp == 1) bw::tmem_dealloc(tmem_base, TMEM_COLS);
}

bool make_map(CUtensorMap* m, const void* base, long long rows, long long K, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    return bw::encode_bf16_sw128(m, base, 2, dims, strides, box);
}

template <bool GATED, typename CT>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const int* tile_expert, void* C, int max_tiles, int N, int K,
           int act, float limit, float alpha, cudaStream_t s) {
    static bool raised[bw::MAX_DEVICES] = {};
    if (cudaError_t e = bw::allow_dynamic_smem(moe_tc_kernel<GATED, CT>, SMEM_BYTES, raised); e != cudaSuccess) return (int)e;
    bw::launch((moe_tc_kernel<GATED, CT>), dim3((N + BN - 1) / BN, max_tiles), dim3(THREADS), SMEM_BYTES, s, ta, tb, tile_expert,
               (CT*)C, N, K, act, limit, alpha);
    BW_LAUNCH_CHECK();
    return 0;
}

}  // namespace

BW_EXPORT int bw_moe_tc_tile_rows() { return BM; }

BW_EXPORT int bw_moe_tc_supported(const void* A, const void* W, int N, int K, int gated) {
    return K > 0 && N > 0 && K % 8 == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0 && (!gated || N % (2 * GATE_BLOCK) == 0);
}

// A: bfloat16 [max_tiles * 128, K]; W: bfloat16 [E, N, K]; tile_expert: int32 [max_tiles].
// gated: W's rows alternate 16 gate / 16 up and C is bfloat16 [rows, N / 2] = glu(gate, up) with the gated
// activation `act` of common.cuh and its limit and alpha (BW_ACT_SILU: silu(gate) * up); else C is [rows, N] of c_type.
BW_EXPORT int bw_moe_gemm_tc(const void* A, const void* W, int gated, const int* tile_expert, void* C, int c_type,
                             int max_tiles, int E, int N, int K, int act, float limit, float alpha, void* stream) {
    if (max_tiles <= 0) return 0;
    if (E <= 0 || !bw_moe_tc_supported(A, W, N, K, gated)) return BW_ERR_UNSUPPORTED;
    if (gated && c_type != BW_BF16) return BW_ERR_BAD_ARG;
    CUtensorMap ta, tb;
    if (!make_map(&ta, A, (long long)max_tiles * BM, K, BM) || !make_map(&tb, W, (long long)E * N, K, BN)) return BW_ERR_DRIVER;
    cudaStream_t s = (cudaStream_t)stream;
    if (gated && act != BW_ACT_SILU && act != BW_ACT_CLAMPED_SWISH) return BW_ERR_BAD_ARG;
    if (gated) return launch<true, bf16>(ta, tb, tile_expert, C, max_tiles, N, K, act, limit, alpha, s);
    if (c_type == BW_F32) return launch<false, float>(ta, tb, tile_expert, C, max_tiles, N, K, 0, 0.f, 1.f, s);
    if (c_type == BW_BF16) return launch<false, bf16>(ta, tb, tile_expert, C, max_tiles, N, K, 0, 0.f, 1.f, s);
    return BW_ERR_BAD_ARG;
}

BW_EXPORT int bw_moe_tc_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
