// Routed experts in prompts on the 5th-generation tensor cores: a grouped product.
//     out[rows of expert e] = X[rows of expert e, K] * W_e[N, K]^T       bfloat16 in, float32 accumulation in tensor memory
// X holds the rows of all experts one after another (gathered and scaled by qnn_moe_gather); the rows of an expert
// are cut into tiles of 128 by qnn_moe_plan, whose tile list (expert, first row) lives on the device, as does their
// number.  The pipeline is that of qnn_gemm_tcgen05 (a persistent CTA per SM, a 4-stage TMA ring, tcgen05.mma from
// shared-memory descriptors into two accumulators in tensor memory, four epilogue warps); what differs:
//   * a tile's rows start at the tile list's row, its weights at row e * N of the stacked matrices (TMA coordinates);
//   * rows of a tile beyond its expert's last row belong to the next expert: they are multiplied and never stored;
//   * the gated epilogue is the clamped one, g' = min(g, limit), u' = clamp(u, -limit, limit),
//     g' * sigmoid(alpha g') * (u' + 1), or, with limit <= 0, the plain silu(g) * u; stored as bfloat16 in the
//     gathered order;
//   * the plain epilogue stores float32 rows back where the rows came from (the permutation), times the row's score
//     when the score goes on the output.
// Every wait on an mbarrier is bounded, as there: when it runs out the thread sets `status` and the CTA still frees
// its tensor memory and returns.
#include "common.cuh"
#include "tcgen05.cuh"

using namespace qnn;

#define EPI_NONE 0
#define EPI_GATED 2
#define EPI_ACT 5               // experts without a gate: out = act(rows w^T), bfloat16 in the gathered order

namespace {

using namespace qnn::tc;
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    umma_bf16_cta1(tmem_d, adesc, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit(unsigned bar) { umma_commit_cta1(bar); }
__device__ __forceinline__ void tmem_ld32(unsigned taddr, uint32_t (&r)[32]) { tmem_ld32_sync(taddr, r); }
inline int make_map(CUtensorMap* map, const void* base, long long rows, long long width, int box_rows) {
    return make_map_bf16(map, base, rows, width, box_rows, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
}

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 256;
constexpr int GEMM_THREADS = 192;

struct __align__(8) Barriers {
    uint64_t full[STAGES];      // a slab has landed (TMA bytes)
    uint64_t empty[STAGES];     // the MMAs that read a slab are done
    uint64_t acc_ready[2];      // an accumulator is complete
    uint64_t acc_free[2];       // the epilogue has read an accumulator out of tensor memory
    uint32_t tmem_base;
    uint32_t failed;
};

__device__ __forceinline__ bool has_failed(Barriers* b) { return *reinterpret_cast<volatile uint32_t*>(&b->failed) != 0; }

// Persistent: a CTA per SM walks over tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (row tiles fastest).
// N: rows of one expert's matrix (gated: gate rows, then as many up rows).
template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS)
moe_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   void* __restrict__ out, int N, int K, const int* __restrict__ offsets, const int* __restrict__ perm,
                   const float* __restrict__ sel_w, const int* __restrict__ tiles, const int* __restrict__ n_row_tiles,
                   int scale_output, float limit, float alpha, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the operand ring wants 1024-byte alignment (8 swizzled rows); the barriers follow it
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    constexpr int OUT_COLS = (EPI == EPI_GATED) ? BN / 2 : BN;          // output columns of a tile
    const int n_tiles = (Nout + OUT_COLS - 1) / OUT_COLS;
    const int nk = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->acc_ready[a]), 1);
            mbar_init(smem_u32(&bars->acc_free[a]), 4);     // one arrival per epilogue warp
        }
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // this warp owns the tensor memory: allocates it here, frees it at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(2 * TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = bars->tmem_base;
    // Barriers and tensor memory are set up; only now wait for the kernels before this one (whose output
    // the loads below read), so that the set-up overlaps their tail.
    pdl_wait();
    const int m_tiles = *n_row_tiles;                        // written by the plan kernel, which has completed by now
    const int ntiles = m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer -------------------------------------------------------------------
            int it = 0;                                    // slabs issued so far, over all tiles
            for (int tile = blockIdx.x; tile < ntiles && !has_failed(bars); tile += gridDim.x) {
                const int rt = tile % m_tiles, n0 = (tile / m_tiles) * OUT_COLS;
                const int e = tiles[2 * rt], m0 = tiles[2 * rt + 1];
                const int w0 = e * N + n0;                 // the expert's rows of the stacked matrices
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(smem_u32(&bars->empty[s]), ((it / STAGES) - 1) & 1)) {
                        atomicOr(status, 1);
                        bars->failed = 1;
                        break;
                    }
                    const unsigned full = smem_u32(&bars->full[s]);
                    const unsigned a_dst = smem_u32(smem + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, full, kb * BK, m0);
                    if (EPI == EPI_GATED) {
                        tma_load_2d(b_dst, &map_b, full, kb * BK, w0);                        // 128 gate rows
                        tma_load_2d(b_dst + B_BYTES / 2, &map_b, full, kb * BK, w0 + Nout);   // the 128 up rows
                    } else {
                        tma_load_2d(b_dst, &map_b, full, kb * BK, w0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue ------------------------------------------------------------
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N >> 3, M >> 4
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
            int it = 0, i = 0;                             // slabs consumed; tiles done by this CTA
            for (int tile = blockIdx.x; tile < ntiles && !has_failed(bars); tile += gridDim.x, ++i) {
                const int a = i & 1;
                if (i >= 2 && !mbar_wait(smem_u32(&bars->acc_free[a]), ((i >> 1) - 1) & 1)) {
                    atomicOr(status, 8);
                    bars->failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned acc = tmem + a * TMEM_COLS;
                bool ok = true;
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&bars->full[s]), (it / STAGES) & 1)) {
                        atomicOr(status, 2);
                        bars->failed = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_addr = smem_u32(smem + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements further along K = 32 bytes inside the 128-byte swizzled row
                        umma_bf16(acc, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bars->empty[s]));     // the stage is free once these MMAs have read it
                }
                umma_commit(smem_u32(&bars->acc_ready[a]));     // arrives when everything issued so far is done
                if (!ok) break;
            }
        }
    } else {
        // ---- epilogue: warps 2..5, each owns the 32 accumulator lanes (rows) of its quarter ----------
        const int quarter = warp & 3;
        int i = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++i) {
            const int a = i & 1;
            const int rt = tile % m_tiles, n0 = (tile / m_tiles) * OUT_COLS;
            const int e = tiles[2 * rt], m0 = tiles[2 * rt + 1];
            const int rows = min(BM, offsets[e + 1] - m0);  // the rest of the tile belongs to the next expert
            if (!mbar_wait(smem_u32(&bars->acc_ready[a]), (i >> 1) & 1)) {
                atomicOr(status, 4);
                bars->failed = 1;
                break;
            }
            if (has_failed(bars)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int r = quarter * 32 + lane;
            int entry = 0;
            float sw = 1.f;
            if (EPI == EPI_NONE && r < rows) {
                entry = perm[m0 + r];
                if (scale_output) sw = sel_w[entry];
            }
            const unsigned lane_addr = tmem + a * TMEM_COLS + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(lane_addr + c0, v);
                float f[32];
                if (EPI == EPI_GATED) {
                    uint32_t u[32];
                    tmem_ld32(lane_addr + BN / 2 + c0, u);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (limit > 0.f) {
                            const float g = fminf(__uint_as_float(v[j]), limit);
                            const float up = fminf(fmaxf(__uint_as_float(u[j]), -limit), limit);
                            f[j] = __fdividef(g, 1.f + __expf(-alpha * g)) * (up + 1.f);
                        } else {                                 // no limit: the plain gate silu(g) * u
                            const float g = __uint_as_float(v[j]);
                            f[j] = __fdividef(g, 1.f + __expf(-g)) * __uint_as_float(u[j]);
                        }
                    }
                } else if (EPI == EPI_ACT) {                     // scale_output carries the activation's code
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = qnn::activate_fast(__uint_as_float(v[j]), scale_output);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * sw;
                }
                if (c0 + 32 >= OUT_COLS) {
                    // the last columns are in registers: hand the accumulator back before storing them
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars->acc_free[a])) : "memory");
                }
                if (r < rows) {
                    if (EPI != EPI_NONE) {
                        bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)(m0 + r) * Nout + n0 + c0;
                        if (n0 + c0 + 32 <= Nout && ((Nout & 7) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) Vec16<bf16>::store(dst + j, f + j);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (n0 + c0 + j < Nout) dst[j] = __float2bfloat16_rn(f[j]);
                        }
                    } else {
                        float* dst = reinterpret_cast<float*>(out) + (size_t)entry * Nout + n0 + c0;
                        if (n0 + c0 + 32 <= Nout && ((Nout & 3) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) Vec16<float>::store(dst + j, f + j);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (n0 + c0 + j < Nout) dst[j] = f[j];
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * TMEM_COLS) : "memory");
    }
}




// gathered[p] = x[row of entry perm[p]] (times the entry's score when the score goes on the input), bfloat16
__global__ void moe_gather_kernel(const bf16* __restrict__ x, int W, const int* __restrict__ perm,
                                  const float* __restrict__ sel_w, int top, int scale_input, bf16* __restrict__ gathered) {
    pdl_wait();
    const int p = blockIdx.x, entry = perm[p];
    const bf16* src = x + (size_t)(entry / top) * W;
    bf16* dst = gathered + (size_t)p * W;
    const float sw = scale_input ? sel_w[entry] : 1.f;
    for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {
        Vec16<bf16> in;
        float v[8];
        in.load(src + i);
        in.unpack(v);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= sw;
        Vec16<bf16>::store(dst + i, v);
    }
}

}  // namespace

QNN_API int qnn_moe_gather(const void* x, int W, const int* perm, const float* sel_w, int top, int scale_input,
                           void* gathered, int n_entries, cudaStream_t st) {
    if (n_entries <= 0) return 0;
    if (W <= 0 || (W & 7) || top <= 0 || ((((uintptr_t)x | (uintptr_t)gathered) & 15) != 0)) return QNN_ERR_UNSUPPORTED;
    qnn::launch_pdl(moe_gather_kernel, dim3(n_entries), dim3(W >= 2048 ? 256 : 128), 0, st, (const bf16*)x, W, perm, sel_w,
                    top, scale_input, (bf16*)gathered);
    QNN_LAUNCH_CHECK();
}

// rows: the gathered rows [n_entries, K] bfloat16; w: [E * N, K] bfloat16, expert after expert.  epi 2: out =
// bfloat16 [n_entries, N / 2] in the gathered order; epi 5: out = act(product), bfloat16 [n_entries, N] in the gathered
// order, the activation's code in `scale_output`; epi 0: out = float32 [n_entries, N], row perm[p] <- gathered row p.
// tiles / n_row_tiles: the plan's list of (expert, first row) for tiles of 128 rows; max_row_tiles bounds it.
QNN_API int qnn_moe_tcgen05(const void* rows, const void* w, void* out, int n_entries, int E, int N, int K, int epi,
                            const int* offsets, const int* perm, const float* sel_w, const int* tiles,
                            const int* n_row_tiles, int max_row_tiles, int scale_output, float limit, float alpha,
                            int* status, cudaStream_t st) {
    if (n_entries <= 0 || max_row_tiles <= 0) return 0;
    if (K <= 0 || (K & 7) || N <= 0 || E <= 0 || ((((uintptr_t)rows | (uintptr_t)w | (uintptr_t)out) & 15) != 0))
        return QNN_ERR_UNSUPPORTED;
    if (epi != EPI_NONE && epi != EPI_GATED && epi != EPI_ACT) return QNN_ERR_ARGUMENT;
    if (epi == EPI_GATED && (N & 1)) return QNN_ERR_ARGUMENT;
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, rows, n_entries, K, BM);
    if (rc) return rc;
    rc = make_map(&map_b, w, (long long)E * N, K, epi == EPI_GATED ? BN / 2 : BN);
    if (rc) return rc;
    const int Nout = epi == EPI_GATED ? N / 2 : N;
    const int cols = epi == EPI_GATED ? BN / 2 : BN;
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
            sm_count = 148;
    }
    const long long ntiles = (long long)max_row_tiles * ((Nout + cols - 1) / cols);
    if (ntiles > 0x7fffffffLL) return QNN_ERR_UNSUPPORTED;
    dim3 grid((unsigned)(ntiles < sm_count ? ntiles : sm_count));
    const size_t smem = (size_t)STAGES * STAGE_BYTES + sizeof(Barriers) + 1024;
    if (epi == EPI_GATED) {
        auto kern = moe_tcgen05_kernel<EPI_GATED>;
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        cudaError_t e = qnn::launch_pdl(kern, grid, dim3(GEMM_THREADS), smem, st, map_a, map_b, out, N, K, offsets, perm,
                                        sel_w, tiles, n_row_tiles, scale_output, limit, alpha, status);
        return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
    }
    if (epi == EPI_ACT) {
        auto kern = moe_tcgen05_kernel<EPI_ACT>;
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        cudaError_t e = qnn::launch_pdl(kern, grid, dim3(GEMM_THREADS), smem, st, map_a, map_b, out, N, K, offsets, perm,
                                        sel_w, tiles, n_row_tiles, scale_output, limit, alpha, status);
        return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
    }
    auto kern = moe_tcgen05_kernel<EPI_NONE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e = qnn::launch_pdl(kern, grid, dim3(GEMM_THREADS), smem, st, map_a, map_b, out, N, K, offsets, perm, sel_w,
                                    tiles, n_row_tiles, scale_output, limit, alpha, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
