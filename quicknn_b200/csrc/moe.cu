// Routed experts, on the device from the router to the sum, so that a decode step stays one CUDA graph.
//
//   qnn_moe_route      router logits (float32 sums), a score function, the `top` best experts of every row
//                      (ties to the lower index) and their scores
//   qnn_moe_plan       rows grouped by expert: offsets, a permutation, and a list of (expert, first row) tiles of
//                      up to 16, 64 or 128 rows; one block
//   qnn_moe_gate_up    per tile: gathered rows (times their score, when the score goes on the input) against the
//                      expert's stacked gate|up matrix, then the gated activation
//   qnn_moe_down       per tile: the expert's down matrix; rows go back to where they came from (float32),
//                      times their score when the score goes on the output
//   qnn_moe_combine    out[t] = sum over a row's experts (+ a shared expert's output), float32
//   qnn_gated_act_clamped   the clamped activation for a dense product: g = min(gate, limit),
//                      u = clamp(up, -limit, limit), g * sigmoid(alpha g) * (u + 1)
//
// The tile kernels: bfloat16 with inner sizes in whole blocks of 32 runs on the tensor cores (mma.sync, 16 or 64 rows
// x 64 output columns per block, weights read as 16-byte operand pieces straight from global memory); everything
// else (float32, other inner sizes) on plain FMA kernels, 16 rows x 128 columns per block, 32 inner elements at a
// time through shared memory.  Sums run over the inner size in a fixed order, so a row's result does not depend on
// which other rows share its tile.
#include "common.cuh"

using namespace qnn;

#define QNN_MOE_SCORE_SIGMOID 0
#define QNN_MOE_SCORE_SOFTMAX 1
#define QNN_GATED_SWIGLU_CLAMPED 2          // after QNN_ACT_GELU_TANH 0 and QNN_ACT_SILU 1

namespace {

constexpr int TILE_ROWS = 16;
constexpr int TILE_COLS = 128;
constexpr int TILE_K = 32;
constexpr int MAX_TOP = 16;

// ---- router ----------------------------------------------------------------------------------------

template <typename TX, typename TW>
__global__ void moe_route_kernel(const TX* __restrict__ x, const TW* __restrict__ wr, int T, int W, int E, int top,
                                 int score_fn, int renorm, const float* __restrict__ correction, float out_scale,
                                 int* __restrict__ sel_e, float* __restrict__ sel_w, int extra,
                                 float* __restrict__ extra_out, int n_groups, int keep_groups) {
    // The matrix may have `extra` rows behind the experts': their products with the row are written to extra_out
    // [T, extra] as they are (float32) and take no part in the choice (a gate's logit formed in the same pass).
    extern __shared__ float sc[];                       // [E] logits (then scores), [E] what the experts are ranked by, [groups]
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int t = blockIdx.x;
    float* s = sc;
    const TX* xr = x + (size_t)t * W;
    // the warps share the experts; a lane's terms and the order of their sum depend on the width only
    constexpr int VX = Vec16<TX>::N, VW = Vec16<TW>::N, V = VX > VW ? VX : VW;
    const bool vec = (W % V) == 0 && ((((uintptr_t)x | (uintptr_t)wr) & 15) == 0);
    for (int e = warp; e < E + extra; e += nwarp) {
        const TW* wrow = wr + (size_t)e * W;
        float d = 0.f;
        if (vec) {
            for (int i = lane * V; i < W; i += 32 * V) {
                float xf[V], wf[V];
#pragma unroll
                for (int j = 0; j < V; j += VX) { Vec16<TX> v; v.load(xr + i + j); v.unpack(xf + j); }
#pragma unroll
                for (int j = 0; j < V; j += VW) { Vec16<TW> v; v.load(wrow + i + j); v.unpack(wf + j); }
#pragma unroll
                for (int j = 0; j < V; ++j) d += xf[j] * wf[j];
            }
        } else {
            for (int i = lane; i < W; i += 32) d += to_f(xr[i]) * to_f(wrow[i]);
        }
        d = warp_sum(d);
        if (lane == 0) {
            if (e < E) s[e] = d;
            else extra_out[(size_t)t * extra + (e - E)] = d;
        }
    }
    __syncthreads();
    if (warp != 0) return;
    __syncwarp();
    // Both score functions rise with the logit, so the experts are chosen by their logits (a sigmoid that has
    // run into 1.0 would tie where the logits still differ) and only the chosen ones' scores are formed.
    float m = -INFINITY, sum = 1.f;
    if (score_fn == QNN_MOE_SCORE_SOFTMAX) {
        for (int e = lane; e < E; e += 32) m = fmaxf(m, s[e]);
        m = warp_max(m);
        sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(s[e] - m);
        sum = warp_sum(sum);
    }
    // With a correction the experts are ranked by score + correction[e] and weighted by the score alone, so every
    // expert's score is formed first.
    float* rank = s;
    const bool ranked = correction != nullptr || n_groups > 1;
    if (ranked) {
        rank = s + E;
        for (int e = lane; e < E; e += 32) {
            const float v = score_fn == QNN_MOE_SCORE_SOFTMAX ? expf(s[e] - m) / sum : 1.f / (1.f + expf(-s[e]));
            s[e] = v;
            rank[e] = v + (correction != nullptr ? correction[e] : 0.f);
        }
        __syncwarp();
    }
    // Groups of neighbouring experts: a group's score is the sum of its two largest ranking values (of its one, where
    // a group is a single expert); only the `keep_groups` best groups stay in the ranking (ties to the lower group),
    // the others' experts rank as minus infinity.
    if (n_groups > 1 && keep_groups < n_groups) {
        float* gs = s + 2 * E;
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;              // the largest and the second
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = rank[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        for (int k = 0; k < keep_groups; ++k) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v > best && v != INFINITY) { best = v; arg = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            __syncwarp();
            if (lane == 0 && arg != 0x7fffffff) gs[arg] = INFINITY;       // kept
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) rank[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = rank[e];
            if (v > best) { best = v; arg = e; }          // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;                    // logits that are all NaN: any expert, the model's logits will show it
        if (ranked) best = s[arg];
        else best = score_fn == QNN_MOE_SCORE_SOFTMAX ? expf(best - m) / sum : 1.f / (1.f + expf(-best));
        total += best;
        __syncwarp();
        if (lane == 0) {
            sel_e[(size_t)t * top + k] = arg;
            sel_w[(size_t)t * top + k] = best;
            rank[arg] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0 && (renorm || out_scale != 1.f))
        for (int k = 0; k < top; ++k) {
            float w = sel_w[(size_t)t * top + k];
            if (renorm) w /= total + 1e-20f;
            sel_w[(size_t)t * top + k] = w * out_scale;
        }
}

// ---- grouping ----------------------------------------------------------------------------------------

// offsets: [E + 1]; perm: [n] sorted place -> entry (row * top + k); tiles: [max_tiles][2] (expert, first sorted
// place); n_tiles: [1].  An entry whose expert id is not in [0, E) belongs to no expert (an identity expert, which
// the combine step serves): it gets no place, and the places behind offsets[E] name entry 0.  Which of an expert's rows comes first varies from run to run; no result depends on it.
__global__ void moe_plan_kernel(const int* __restrict__ sel_e, int n, int E, int tile_rows, int* __restrict__ offsets,
                                int* __restrict__ perm, int* __restrict__ tiles, int* __restrict__ n_tiles) {
    extern __shared__ int cnt[];                        // [E] counts, then [E] running places
    int* at = cnt + E;
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        if ((unsigned)sel_e[i] < (unsigned)E) atomicAdd(&cnt[sel_e[i]], 1);
    __syncthreads();
    __shared__ int placed;
    if (threadIdx.x == 0) {
        int o = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = o;
            at[e] = o;
            for (int r = 0; r < cnt[e]; r += tile_rows) {
                tiles[2 * nt] = e;
                tiles[2 * nt + 1] = o + r;
                ++nt;
            }
            o += cnt[e];
        }
        offsets[E] = o;
        *n_tiles = nt;
        placed = o;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        if ((unsigned)sel_e[i] < (unsigned)E) perm[atomicAdd(&at[sel_e[i]], 1)] = i;
    for (int i = placed + threadIdx.x; i < n; i += blockDim.x) perm[i] = 0;
}

// ---- tiles ---------------------------------------------------------------------------------------------

__device__ __forceinline__ float gated(float g, float u, int act, float limit, float alpha) {
    if (act == QNN_GATED_SWIGLU_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g * (1.f / (1.f + expf(-alpha * g))) * (u + 1.f);
    }
    return activate(g, act) * u;
}

// acc[m][r] += sum_k xs[k][r] * w_m[col][k] over K, for NM matrices whose rows `col` lie `K` apart.
// xs is filled by `fill(k0, kn)` for each block of inner elements.
template <typename TW, int NM, typename Fill>
__device__ __forceinline__ void tile_product(const TW* const* w, int col0, int n_cols, int K, float (*xs)[TILE_ROWS],
                                             float (*ws)[TILE_K][TILE_COLS + 1], float (&acc)[NM][TILE_ROWS], Fill fill) {
    for (int k0 = 0; k0 < K; k0 += TILE_K) {
        const int kn = min(TILE_K, K - k0);
        __syncthreads();
        fill(k0, kn);
#pragma unroll
        for (int m = 0; m < NM; ++m)
            for (int idx = threadIdx.x; idx < TILE_COLS * TILE_K; idx += TILE_COLS) {
                const int c = idx / TILE_K, kk = idx - c * TILE_K;
                ws[m][kk][c] = (c < n_cols && kk < kn) ? to_f(w[m][(size_t)(col0 + c) * K + k0 + kk]) : 0.f;
            }
        __syncthreads();
#pragma unroll 4
        for (int kk = 0; kk < TILE_K; ++kk) {
            float xv[TILE_ROWS];
#pragma unroll
            for (int r = 0; r < TILE_ROWS; r += 4) {
                const float4 f = *reinterpret_cast<const float4*>(&xs[kk][r]);
                xv[r] = f.x; xv[r + 1] = f.y; xv[r + 2] = f.z; xv[r + 3] = f.w;
            }
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                const float wv = ws[m][kk][threadIdx.x];
#pragma unroll
                for (int r = 0; r < TILE_ROWS; ++r) acc[m][r] += xv[r] * wv;
            }
        }
    }
}

// NM = 2: the expert's matrix holds gate rows, then up rows, and the result is act(gate) * up; NM = 1: up rows alone,
// and the result is act(up).
template <typename T, int NM>
__global__ void __launch_bounds__(TILE_COLS)
moe_gate_up_kernel(const T* __restrict__ x, int W, const T* __restrict__ w_gu, int ff, const int* __restrict__ offsets,
                   const int* __restrict__ perm, const float* __restrict__ sel_w, const int* __restrict__ tiles,
                   const int* __restrict__ n_tiles, int top, int scale_input, int act, float limit, float alpha,
                   T* __restrict__ hidden) {
    __shared__ __align__(16) float xs[TILE_K][TILE_ROWS];
    __shared__ float ws[NM][TILE_K][TILE_COLS + 1];
    __shared__ int src_row[TILE_ROWS];
    __shared__ float src_w[TILE_ROWS];
    pdl_wait();
    if ((int)blockIdx.x >= *n_tiles) return;
    const int e = tiles[2 * blockIdx.x], p0 = tiles[2 * blockIdx.x + 1];
    const int rows = min(TILE_ROWS, offsets[e + 1] - p0);
    const int col0 = blockIdx.y * TILE_COLS, n_cols = min(TILE_COLS, ff - col0);
    if (threadIdx.x < TILE_ROWS) {
        const int entry = threadIdx.x < rows ? perm[p0 + threadIdx.x] : -1;
        src_row[threadIdx.x] = entry < 0 ? -1 : entry / top;
        src_w[threadIdx.x] = (entry < 0 || !scale_input) ? 1.f : sel_w[entry];
    }
    const T* wg = w_gu + (size_t)e * NM * ff * W;
    const T* w2[NM];
#pragma unroll
    for (int m = 0; m < NM; ++m) w2[m] = wg + (size_t)m * ff * W;
    float acc[NM][TILE_ROWS];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int r = 0; r < TILE_ROWS; ++r) acc[m][r] = 0.f;
    tile_product<T, NM>(w2, col0, n_cols, W, xs, ws, acc, [&](int k0, int kn) {
        for (int idx = threadIdx.x; idx < TILE_ROWS * TILE_K; idx += TILE_COLS) {
            const int r = idx / TILE_K, kk = idx - r * TILE_K;
            const int row = src_row[r];
            xs[kk][r] = (row >= 0 && kk < kn) ? to_f(x[(size_t)row * W + k0 + kk]) * src_w[r] : 0.f;
        }
    });
    if ((int)threadIdx.x < n_cols)
        for (int r = 0; r < rows; ++r)
            hidden[(size_t)(p0 + r) * ff + col0 + threadIdx.x] =
                from_f<T>(NM == 2 ? gated(acc[0][r], acc[NM - 1][r], act, limit, alpha) : activate(acc[0][r], act));
}

template <typename T>
__global__ void __launch_bounds__(TILE_COLS)
moe_down_kernel(const T* __restrict__ hidden, int ff, const T* __restrict__ w_down, int W, const int* __restrict__ offsets,
                const int* __restrict__ perm, const float* __restrict__ sel_w, const int* __restrict__ tiles,
                const int* __restrict__ n_tiles, int scale_output, float* __restrict__ ys) {
    __shared__ __align__(16) float xs[TILE_K][TILE_ROWS];
    __shared__ float ws[1][TILE_K][TILE_COLS + 1];
    pdl_wait();
    if ((int)blockIdx.x >= *n_tiles) return;
    const int e = tiles[2 * blockIdx.x], p0 = tiles[2 * blockIdx.x + 1];
    const int rows = min(TILE_ROWS, offsets[e + 1] - p0);
    const int col0 = blockIdx.y * TILE_COLS, n_cols = min(TILE_COLS, W - col0);
    const T* const w1[1] = {w_down + (size_t)e * W * ff};
    float acc[1][TILE_ROWS];
#pragma unroll
    for (int r = 0; r < TILE_ROWS; ++r) acc[0][r] = 0.f;
    tile_product<T, 1>(w1, col0, n_cols, ff, xs, ws, acc, [&](int k0, int kn) {
        for (int idx = threadIdx.x; idx < TILE_ROWS * TILE_K; idx += TILE_COLS) {
            const int r = idx / TILE_K, kk = idx - r * TILE_K;
            xs[kk][r] = (r < rows && kk < kn) ? to_f(hidden[(size_t)(p0 + r) * ff + k0 + kk]) : 0.f;
        }
    });
    if ((int)threadIdx.x < n_cols)
        for (int r = 0; r < rows; ++r) {
            const int entry = perm[p0 + r];
            ys[(size_t)entry * W + col0 + threadIdx.x] = acc[0][r] * (scale_output ? sel_w[entry] : 1.f);
        }
}

// ---- the same tiles on the tensor cores (bfloat16) -----------------------------------------------------------------
// A block owns MT x 16 rows of one expert and 64 output columns (4 warps x 2 column tiles of 8).  The rows' activations
// pass through shared memory 256 inner elements at a time; the weights never do: a lane reads 16 bytes of a weight
// row straight into the B operand.  That is possible because a sum over the inner index may run in any order: within
// a block of 32 inner elements lane (g, tg) takes elements 8 tg .. 8 tg + 7 of weight row g, which are the B pairs
// of two m16n8k16 steps, and the A operand takes the same elements of the activation rows (one 16-byte load from
// shared memory per row half).  Sums are float32; a row's result does not depend on the other rows of its tile.

constexpr int MMA_WARPS = 4, MMA_NW = 2, MMA_COLS = MMA_WARPS * MMA_NW * 8, MMA_KC = 256, MMA_PITCH = MMA_KC + 32;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// acc[m][t][j] += rows x weights over K (a multiple of 32) for NM matrices; `fill(k0, kn)` puts the rows' elements
// k0 .. k0 + kn - 1 into xs ([MT*16][MMA_PITCH] bfloat16, zero rows beyond the tile's).
template <int MT, int NM, typename Fill>
__device__ __forceinline__ void mma_tile_product(const bf16* const* w, int col0, int n_cols, int K, bf16* xs,
                                                 float (&acc)[NM][MT][MMA_NW][4], Fill fill) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
    const bf16* wrow[NM][MMA_NW];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int t = 0; t < MMA_NW; ++t) {
            const int c = min((warp * MMA_NW + t) * 8 + g, n_cols - 1);          // columns beyond the matrix: any row, unused
            wrow[m][t] = w[m] + (size_t)(col0 + c) * K + 8 * tg;
        }
    for (int k0 = 0; k0 < K; k0 += MMA_KC) {
        const int kn = min(MMA_KC, K - k0);
        __syncthreads();
        fill(k0, kn);
        __syncthreads();
        uint4 bnext[NM][MMA_NW];
#pragma unroll
        for (int m = 0; m < NM; ++m)
#pragma unroll
            for (int t = 0; t < MMA_NW; ++t) bnext[m][t] = *reinterpret_cast<const uint4*>(wrow[m][t] + k0);
        for (int kb = 0; kb < kn; kb += 32) {
            uint4 b[NM][MMA_NW];
#pragma unroll
            for (int m = 0; m < NM; ++m)
#pragma unroll
                for (int t = 0; t < MMA_NW; ++t) {
                    b[m][t] = bnext[m][t];
                    if (kb + 32 < kn) bnext[m][t] = *reinterpret_cast<const uint4*>(wrow[m][t] + k0 + kb + 32);
                }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint4 lo = *reinterpret_cast<const uint4*>(xs + (size_t)(mt * 16 + g) * MMA_PITCH + kb + 8 * tg);
                const uint4 hi = *reinterpret_cast<const uint4*>(xs + (size_t)(mt * 16 + g + 8) * MMA_PITCH + kb + 8 * tg);
#pragma unroll
                for (int m = 0; m < NM; ++m)
#pragma unroll
                    for (int t = 0; t < MMA_NW; ++t) {
                        mma_bf16(acc[m][mt][t], lo.x, hi.x, lo.y, hi.y, b[m][t].x, b[m][t].y);
                        mma_bf16(acc[m][mt][t], lo.z, hi.z, lo.w, hi.w, b[m][t].z, b[m][t].w);
                    }
            }
        }
    }
}

template <int MT, int NM>
__global__ void __launch_bounds__(MMA_WARPS * 32)
moe_gate_up_mma_kernel(const bf16* __restrict__ x, int W, const bf16* __restrict__ w_gu, int ff,
                       const int* __restrict__ offsets, const int* __restrict__ perm, const float* __restrict__ sel_w,
                       const int* __restrict__ tiles, const int* __restrict__ n_tiles, int top, int scale_input, int act,
                       float limit, float alpha, bf16* __restrict__ hidden) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);
    __shared__ int src_row[MT * 16];
    __shared__ float src_w[MT * 16];
    pdl_wait();
    if ((int)blockIdx.x >= *n_tiles) return;
    const int e = tiles[2 * blockIdx.x], p0 = tiles[2 * blockIdx.x + 1];
    const int rows = min(MT * 16, offsets[e + 1] - p0);
    const int col0 = blockIdx.y * MMA_COLS, n_cols = min(MMA_COLS, ff - col0);
    for (int r = threadIdx.x; r < MT * 16; r += blockDim.x) {
        const int entry = r < rows ? perm[p0 + r] : -1;
        src_row[r] = entry < 0 ? -1 : entry / top;
        src_w[r] = (entry < 0 || !scale_input) ? 1.f : sel_w[entry];
    }
    const bf16* wg = w_gu + (size_t)e * NM * ff * W;
    const bf16* w2[NM];
#pragma unroll
    for (int m = 0; m < NM; ++m) w2[m] = wg + (size_t)m * ff * W;
    float acc[NM][MT][MMA_NW][4] = {};
    mma_tile_product<MT, NM>(w2, col0, n_cols, W, xs, acc, [&](int k0, int kn) {
        for (int idx = threadIdx.x; idx < MT * 16 * (MMA_KC / 8); idx += blockDim.x) {
            const int r = idx / (MMA_KC / 8), kk = (idx - r * (MMA_KC / 8)) * 8;
            const int row = src_row[r];
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (row >= 0 && kk < kn) {
                Vec16<bf16> in;
                in.load(x + (size_t)row * W + k0 + kk);
                in.unpack(v);
                const float sw = src_w[r];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= sw;
            }
            Vec16<bf16>::store(xs + (size_t)r * MMA_PITCH + kk, v);
        }
    });
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int t = 0; t < MMA_NW; ++t)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = mt * 16 + g + (j >> 1) * 8, c = (warp * MMA_NW + t) * 8 + 2 * tg + (j & 1);
                if (r < rows && c < n_cols)
                    hidden[(size_t)(p0 + r) * ff + col0 + c] =
                        __float2bfloat16_rn(NM == 2 ? gated(acc[0][mt][t][j], acc[NM - 1][mt][t][j], act, limit, alpha)
                                                    : activate(acc[0][mt][t][j], act));
            }
}

template <int MT>
__global__ void __launch_bounds__(MMA_WARPS * 32)
moe_down_mma_kernel(const bf16* __restrict__ hidden, int ff, const bf16* __restrict__ w_down, int W,
                    const int* __restrict__ offsets, const int* __restrict__ perm, const float* __restrict__ sel_w,
                    const int* __restrict__ tiles, const int* __restrict__ n_tiles, int scale_output,
                    float* __restrict__ ys) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);
    pdl_wait();
    if ((int)blockIdx.x >= *n_tiles) return;
    const int e = tiles[2 * blockIdx.x], p0 = tiles[2 * blockIdx.x + 1];
    const int rows = min(MT * 16, offsets[e + 1] - p0);
    const int col0 = blockIdx.y * MMA_COLS, n_cols = min(MMA_COLS, W - col0);
    const bf16* const w1[1] = {w_down + (size_t)e * W * ff};
    float acc[1][MT][MMA_NW][4] = {};
    mma_tile_product<MT, 1>(w1, col0, n_cols, ff, xs, acc, [&](int k0, int kn) {
        for (int idx = threadIdx.x; idx < MT * 16 * (MMA_KC / 8); idx += blockDim.x) {
            const int r = idx / (MMA_KC / 8), kk = (idx - r * (MMA_KC / 8)) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows && kk < kn) v = *reinterpret_cast<const uint4*>(hidden + (size_t)(p0 + r) * ff + k0 + kk);
            *reinterpret_cast<uint4*>(xs + (size_t)r * MMA_PITCH + kk) = v;
        }
    });
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = mt * 16 + g + (j >> 1) * 8;
            if (r >= rows) continue;
            const int entry = perm[p0 + r];
            const float sw = scale_output ? sel_w[entry] : 1.f;
#pragma unroll
            for (int t = 0; t < MMA_NW; ++t) {
                const int c = (warp * MMA_NW + t) * 8 + 2 * tg + (j & 1);
                if (c < n_cols) ys[(size_t)entry * W + col0 + c] = acc[0][mt][t][j] * sw;
            }
        }
}

inline bool mma_takes(int dtype, int K, const void* a, const void* b) {
    return dtype == QNN_DT_BF16 && K % 32 == 0 && ((((uintptr_t)a | (uintptr_t)b) & 15) == 0);
}

// out[t] = sum over the row's entries of the expert's output, or, for an entry whose expert id is E or more (an
// identity expert), of its score times the row x[t] itself; plus the shared expert's output, times
// sigmoid(shared_gate[t]) when the shared expert has a gate.
__global__ void moe_combine_kernel(const float* __restrict__ ys, int top, const void* __restrict__ shared, int shared_dt,
                                   const float* __restrict__ shared_gate, const int* __restrict__ sel_e,
                                   const float* __restrict__ sel_w, int E, const void* __restrict__ x, int x_dt,
                                   float* __restrict__ out, int W, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / W, c = i - t * W;
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
        if (sel_e != nullptr && sel_e[t * top + k] >= E) s += sel_w[t * top + k] * load_as_f(x, x_dt, i);
        else s += ys[(t * top + k) * W + c];
    }
    if (shared) {
        const float v = load_as_f(shared, shared_dt, i);
        s += shared_gate != nullptr ? v * (1.f / (1.f + expf(-shared_gate[t]))) : v;
    }
    out[i] = s;
}

template <typename T>
__global__ void gated_act_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, float limit, float alpha,
                                         size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / I, c = i - t * I;
    out[i] = from_f<T>(gated(to_f(gu[t * 2 * I + c]), to_f(gu[t * 2 * I + I + c]), QNN_GATED_SWIGLU_CLAMPED, limit, alpha));
}

}  // namespace

QNN_API int qnn_moe_route(const void* x, int x_dt, const void* w_router, int w_dt, int T, int W, int E, int top,
                          int score_fn, int renorm, const float* correction, float out_scale, int* sel_e, float* sel_w,
                          int extra, float* extra_out, int n_groups, int keep_groups, cudaStream_t st) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || top > MAX_TOP || W <= 0) return QNN_ERR_ARGUMENT;
    if (extra < 0 || (extra > 0 && extra_out == nullptr)) return QNN_ERR_ARGUMENT;
    // groups: equal groups of neighbours, and enough experts in the kept groups for the choice
    if (n_groups < 1) n_groups = keep_groups = 1;
    if (E % n_groups || keep_groups < 1 || keep_groups > n_groups || (long long)keep_groups * (E / n_groups) < top)
        return QNN_ERR_ARGUMENT;
    const int warps = E >= 8 ? 8 : (E >= 4 ? 4 : 2);
    const size_t smem = ((size_t)2 * E + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return QNN_ERR_UNSUPPORTED;
    const dim3 grid(T), block(warps * 32);
#define QNN_ROUTE(TX, TW)                                                                                         \
    launch_pdl(moe_route_kernel<TX, TW>, grid, block, smem, st, (const TX*)x, (const TW*)w_router, T, W, E, top,  \
               score_fn, renorm, correction, out_scale, sel_e, sel_w, extra, extra_out, n_groups, keep_groups)
    if (x_dt == QNN_DT_BF16 && w_dt == QNN_DT_BF16) QNN_ROUTE(bf16, bf16);
    else if (x_dt == QNN_DT_BF16) QNN_ROUTE(bf16, float);
    else if (w_dt == QNN_DT_BF16) QNN_ROUTE(float, bf16);
    else QNN_ROUTE(float, float);
#undef QNN_ROUTE
    QNN_LAUNCH_CHECK();
}

// Rows of a tile: 16, or 64 where the experts get many rows each and the two matrices take the tensor-core kernel
// (a tile's weights are then read once for four times the rows).
QNN_API int qnn_moe_tile_rows(int n_entries, int E, int dtype, int W, int ff) {
    const bool mma = dtype == QNN_DT_BF16 && W % 32 == 0 && ff % 32 == 0;
    return (mma && n_entries >= 48 * E) ? 64 : TILE_ROWS;
}
QNN_API int qnn_moe_max_tiles(int n_entries, int E, int tile_rows) { return (n_entries + tile_rows - 1) / tile_rows + E; }

QNN_API int qnn_moe_plan(const int* sel_e, int n, int E, int tile_rows, int* offsets, int* perm, int* tiles, int* n_tiles,
                         cudaStream_t st) {
    if (n <= 0) return 0;
    if (E <= 0 || (size_t)2 * E * sizeof(int) > 48 * 1024 || (tile_rows != 16 && tile_rows != 64 && tile_rows != 128))
        return QNN_ERR_ARGUMENT;
    launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), st, sel_e, n, E, tile_rows, offsets, perm,
               tiles, n_tiles);
    QNN_LAUNCH_CHECK();
}

// act: the gate's activation (QNN_ACT_GELU_TANH, QNN_ACT_SILU or QNN_GATED_SWIGLU_CLAMPED); with QNN_ACT_ALONE added the
// experts have no gate: w_gu is [E, ff, W] (up rows alone) and hidden = act(up(x)), act any QNN_ACT_* code.
QNN_API int qnn_moe_gate_up(const void* x, int dtype, int W, const void* w_gu, int ff, const int* offsets, const int* perm,
                            const float* sel_w, const int* tiles, const int* n_tiles, int max_tiles, int tile_rows,
                            int top, int scale_input, int act, float limit, float alpha, void* hidden, cudaStream_t st) {
    if (max_tiles <= 0) return 0;
    if (W <= 0 || ff <= 0 || top <= 0) return QNN_ERR_ARGUMENT;
    if (tile_rows != 16 && tile_rows != 64) return QNN_ERR_ARGUMENT;
    const bool alone = (act & QNN_ACT_ALONE) != 0;
    act &= ~QNN_ACT_ALONE;
    if (mma_takes(dtype, W, x, w_gu)) {
        const dim3 mgrid(max_tiles, (ff + MMA_COLS - 1) / MMA_COLS);
        if (mgrid.y > 65535) return QNN_ERR_UNSUPPORTED;
        const size_t smem = (size_t)tile_rows * MMA_PITCH * sizeof(bf16);
#define QNN_GU_MMA(MT, NM)                                                                                             \
        {                                                                                                              \
            static bool set = false;                                                                                   \
            if (smem > 48 * 1024 && !set) {                                                                            \
                cudaFuncSetAttribute(moe_gate_up_mma_kernel<MT, NM>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                     (int)smem);                                                                       \
                set = true;                                                                                            \
            }                                                                                                          \
            launch_pdl(moe_gate_up_mma_kernel<MT, NM>, mgrid, dim3(MMA_WARPS * 32), smem, st, (const bf16*)x, W,      \
                       (const bf16*)w_gu, ff, offsets, perm, sel_w, tiles, n_tiles, top, scale_input, act, limit,      \
                       alpha, (bf16*)hidden);                                                                          \
        }
        if (tile_rows == 64) {
            if (alone) QNN_GU_MMA(4, 1) else QNN_GU_MMA(4, 2)
        } else {
            if (alone) QNN_GU_MMA(1, 1) else QNN_GU_MMA(1, 2)
        }
#undef QNN_GU_MMA
        QNN_LAUNCH_CHECK();
    }
    if (tile_rows != TILE_ROWS) return QNN_ERR_ARGUMENT;
    const dim3 grid(max_tiles, (ff + TILE_COLS - 1) / TILE_COLS);
    if (grid.y > 65535) return QNN_ERR_UNSUPPORTED;
#define QNN_GU(T, NM)                                                                                                  \
    launch_pdl(moe_gate_up_kernel<T, NM>, grid, dim3(TILE_COLS), 0, st, (const T*)x, W, (const T*)w_gu, ff, offsets,  \
               perm, sel_w, tiles, n_tiles, top, scale_input, act, limit, alpha, (T*)hidden)
    if (dtype == QNN_DT_BF16) {
        if (alone) QNN_GU(bf16, 1); else QNN_GU(bf16, 2);
    } else {
        if (alone) QNN_GU(float, 1); else QNN_GU(float, 2);
    }
#undef QNN_GU
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_moe_down(const void* hidden, int dtype, int ff, const void* w_down, int W, const int* offsets,
                         const int* perm, const float* sel_w, const int* tiles, const int* n_tiles, int max_tiles,
                         int tile_rows, int scale_output, float* ys, cudaStream_t st) {
    if (max_tiles <= 0) return 0;
    if (W <= 0 || ff <= 0) return QNN_ERR_ARGUMENT;
    if (tile_rows != 16 && tile_rows != 64) return QNN_ERR_ARGUMENT;
    if (mma_takes(dtype, ff, hidden, w_down)) {
        const dim3 mgrid(max_tiles, (W + MMA_COLS - 1) / MMA_COLS);
        if (mgrid.y > 65535) return QNN_ERR_UNSUPPORTED;
        const size_t smem = (size_t)tile_rows * MMA_PITCH * sizeof(bf16);
        if (tile_rows == 64) {
            static bool set = false;
            if (!set) {
                cudaFuncSetAttribute(moe_down_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                set = true;
            }
            launch_pdl(moe_down_mma_kernel<4>, mgrid, dim3(MMA_WARPS * 32), smem, st, (const bf16*)hidden, ff,
                       (const bf16*)w_down, W, offsets, perm, sel_w, tiles, n_tiles, scale_output, ys);
        } else {
            launch_pdl(moe_down_mma_kernel<1>, mgrid, dim3(MMA_WARPS * 32), smem, st, (const bf16*)hidden, ff,
                       (const bf16*)w_down, W, offsets, perm, sel_w, tiles, n_tiles, scale_output, ys);
        }
        QNN_LAUNCH_CHECK();
    }
    if (tile_rows != TILE_ROWS) return QNN_ERR_ARGUMENT;
    const dim3 grid(max_tiles, (W + TILE_COLS - 1) / TILE_COLS);
    if (grid.y > 65535) return QNN_ERR_UNSUPPORTED;
    if (dtype == QNN_DT_BF16)
        launch_pdl(moe_down_kernel<bf16>, grid, dim3(TILE_COLS), 0, st, (const bf16*)hidden, ff, (const bf16*)w_down, W,
                   offsets, perm, sel_w, tiles, n_tiles, scale_output, ys);
    else
        launch_pdl(moe_down_kernel<float>, grid, dim3(TILE_COLS), 0, st, (const float*)hidden, ff, (const float*)w_down, W,
                   offsets, perm, sel_w, tiles, n_tiles, scale_output, ys);
    QNN_LAUNCH_CHECK();
}

// sel_e, sel_w, E, x: given when some expert ids may be E or more (identity experts); null / 0 otherwise.
QNN_API int qnn_moe_combine(const float* ys, int top, const void* shared, int shared_dt, const float* shared_gate,
                            const int* sel_e, const float* sel_w, int E, const void* x, int x_dt, float* out, int T, int W,
                            cudaStream_t st) {
    if (T <= 0) return 0;
    if (sel_e != nullptr && (sel_w == nullptr || x == nullptr)) return QNN_ERR_ARGUMENT;
    const size_t n = (size_t)T * W;
    launch_pdl(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, ys, top, shared, shared_dt,
               shared_gate, sel_e, sel_w, E, x, x_dt, out, W, n);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_gated_act_clamped(const void* gu, void* out, int dtype, int T, int I, float limit, float alpha,
                                  cudaStream_t st) {
    if (T <= 0) return 0;
    const size_t n = (size_t)T * I;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == QNN_DT_BF16)
        launch_pdl(gated_act_clamped_kernel<bf16>, grid, dim3(256), 0, st, (const bf16*)gu, (bf16*)out, I, limit, alpha, n);
    else
        launch_pdl(gated_act_clamped_kernel<float>, grid, dim3(256), 0, st, (const float*)gu, (float*)out, I, limit, alpha,
                   n);
    QNN_LAUNCH_CHECK();
}
