// Parts of layers whose sublayers run side by side on one normed input, and of norms taken in groups.
//
//   qnn_group_rmsnorm        RMS norm in groups: a row of H columns is cut into `groups` equal consecutive pieces, each
//                            is divided by its own sqrt(mean(piece^2) + eps), and the whole is multiplied by w [H]
//   qnn_add2_group_rmsnorm   resid += a + b (either may be absent; element types of their own) and, optionally, the
//                            grouped norm of the new stream in the same kernel: what a layer with parallel sublayers
//                            does at its end, together with the first norm of the layer that follows
//   qnn_embed_pos            out[t] = table[token_t] * scale + pos_table[position_t], optionally with the grouped norm
//                            of that row in the same kernel (a learned position vector per position)
//   qnn_sigmoid_gate         o[t, c] *= sigmoid(g[t, c]): a gate per element, rows with pitches of their own
//   qnn_xielu                x > 0: ap x^2 + x / 2;  x <= 0: an (exp(x) - 1 - x) + x / 2
//
// Sums are float32; a group's sum is formed by the same threads in the same order whatever else the batch holds.
#include "common.cuh"

#include <initializer_list>

using namespace qnn;

namespace {

constexpr int NORM_THREADS = 256;
constexpr int NORM_WARPS = NORM_THREADS / 32;

// Warps of a block that share one group: all of them for one group, half for two, ... one from eight groups on.
__device__ __forceinline__ int warps_per_group(int groups) {
    int w = NORM_WARPS;
    while (w > 1 && NORM_WARPS / w < groups) w >>= 1;
    return w;
}

// The grouped norm of row[0 .. H) (float32, in global or shared memory; every thread sees what it needs of it):
// teams of `wpg` warps take the groups in turn.  red: NORM_WARPS floats of shared memory.  VEC: a thread takes eight
// consecutive columns at a time with 16-byte accesses (groups of whole eights, every base on 16 bytes).
template <bool VEC>
__device__ __forceinline__ void group_norm_row(const float* row, int H, int groups, const void* __restrict__ w, int w_dt,
                                               float eps, void* __restrict__ out, int out_dt, size_t out_base,
                                               float* red) {
    constexpr int STEP = VEC ? 8 : 1;
    const int gs = H / groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpg = warps_per_group(groups), teams = NORM_WARPS / wpg;
    const int team = warp / wpg, in_team = (warp % wpg) * 32 + lane, team_threads = wpg * 32;
    for (int g0 = 0; g0 < groups; g0 += teams) {
        const int g = g0 + team;
        const bool live = g < groups;
        float ss = 0.f;
        if (live)
            for (int i = in_team * STEP; i < gs; i += team_threads * STEP) {
                if (VEC) {
                    const float4 a = *reinterpret_cast<const float4*>(row + (size_t)g * gs + i);
                    const float4 b = *reinterpret_cast<const float4*>(row + (size_t)g * gs + i + 4);
                    ss += (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w) + (b.x * b.x + b.y * b.y) + (b.z * b.z + b.w * b.w);
                } else {
                    const float v = row[(size_t)g * gs + i];
                    ss += v * v;
                }
            }
        ss = warp_sum(ss);
        if (wpg > 1) {
            __syncthreads();
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            ss = 0.f;
            for (int k = 0; k < wpg; ++k) ss += red[team * wpg + k];
        }
        if (live) {
            const float inv = rsqrtf(ss / (float)gs + eps);
            for (int i = in_team * STEP; i < gs; i += team_threads * STEP) {
                const size_t c = (size_t)g * gs + i;
                if (VEC) {
                    float wv[8], o[8];
                    load8_as_f(w, w_dt, c, wv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[e] = row[c + e] * inv * wv[e];
                    store8_from_f(out, out_dt, out_base + c, o);
                } else {
                    store_from_f(out, out_dt, out_base + c, row[c] * inv * load_as_f(w, w_dt, c));
                }
            }
        }
    }
}

template <bool VEC>
__global__ void __launch_bounds__(NORM_THREADS)
group_rmsnorm_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ w, int w_dt, float eps, int groups,
                     void* __restrict__ out, int out_dt, int H) {
    extern __shared__ __align__(16) float row[];    // [H], then NORM_WARPS
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    if (VEC) {
        for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) load8_as_f(x, x_dt, base + i, row + i);
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = load_as_f(x, x_dt, base + i);
    }
    __syncthreads();
    group_norm_row<VEC>(row, H, groups, w, w_dt, eps, out, out_dt, base, row + H);
}

template <bool VEC>
__global__ void __launch_bounds__(NORM_THREADS)
add2_group_rmsnorm_kernel(float* __restrict__ resid, const void* __restrict__ a, int a_dt, const void* __restrict__ b,
                          int b_dt, const void* __restrict__ w, int w_dt, float eps, int groups, void* __restrict__ out,
                          int out_dt, int H) {
    extern __shared__ __align__(16) float row[];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    if (VEC) {
        for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
            float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, z[8], r[8];
            if (a != nullptr) load8_as_f(a, a_dt, base + i, y);
            if (b != nullptr) {
                load8_as_f(b, b_dt, base + i, z);
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] += z[e];
            }
            load8_as_f(resid, QNN_DT_F32, base + i, r);
#pragma unroll
            for (int e = 0; e < 8; ++e) r[e] += y[e];          // the sublayers' sum first, then the stream
            store8_from_f(resid, QNN_DT_F32, base + i, r);
#pragma unroll
            for (int e = 0; e < 8; ++e) row[i + e] = r[e];
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float y = a != nullptr ? load_as_f(a, a_dt, base + i) : 0.f;
            if (b != nullptr) y += load_as_f(b, b_dt, base + i);
            const float v = resid[base + i] + y;               // the sublayers' sum first, then the stream
            resid[base + i] = v;
            row[i] = v;
        }
    }
    if (out == nullptr) return;
    __syncthreads();
    group_norm_row<VEC>(row, H, groups, w, w_dt, eps, out, out_dt, base, row + H);
}

template <bool VEC>
__global__ void __launch_bounds__(NORM_THREADS)
embed_pos_kernel(const int* __restrict__ tokens, const void* __restrict__ table, int t_dt, float scale,
                 const void* __restrict__ pos_table, int p_dt, const int* __restrict__ tok_pos, int n_pos,
                 float* __restrict__ out, const void* __restrict__ w, int w_dt, float eps, int groups,
                 void* __restrict__ normed, int n_dt, int H, int V) {
    extern __shared__ __align__(16) float row[];
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t], p = tok_pos[t];
    const bool tv = tok >= 0 && tok < V, pv = p >= 0 && p < n_pos;
    const size_t base = (size_t)t * H;
    if (VEC) {
        for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, z[8];
            if (tv) {
                load8_as_f(table, t_dt, (size_t)tok * H + i, v);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] *= scale;
            }
            if (pv) {
                load8_as_f(pos_table, p_dt, (size_t)p * H + i, z);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += z[e];
            }
            store8_from_f(out, QNN_DT_F32, base + i, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) row[i + e] = v[e];
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = tv ? load_as_f(table, t_dt, (size_t)tok * H + i) * scale : 0.f;
            if (pv) v += load_as_f(pos_table, p_dt, (size_t)p * H + i);
            out[base + i] = v;
            row[i] = v;
        }
    }
    if (normed == nullptr) return;
    __syncthreads();
    group_norm_row<VEC>(row, H, groups, w, w_dt, eps, normed, n_dt, base, row + H);
}

template <bool VEC>
__global__ void sigmoid_gate_kernel(void* __restrict__ o, int o_dt, long long ldo, const void* __restrict__ g, int g_dt,
                                    long long ldg, int N, int accurate) {
    pdl_wait();
    const size_t ob = (size_t)blockIdx.x * ldo, gb = (size_t)blockIdx.x * ldg;
    if (VEC) {
        for (int i = threadIdx.x * 8; i < N; i += blockDim.x * 8) {
            float z[8], v[8];
            load8_as_f(g, g_dt, gb + i, z);
            load8_as_f(o, o_dt, ob + i, v);
#pragma unroll
            for (int e = 0; e < 8; ++e)
                v[e] *= accurate ? 1.f / (1.f + expf(-z[e])) : __fdividef(1.f, 1.f + __expf(-z[e]));
            store8_from_f(o, o_dt, ob + i, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float z = load_as_f(g, g_dt, gb + i);
        const float s = accurate ? 1.f / (1.f + expf(-z)) : __fdividef(1.f, 1.f + __expf(-z));
        store_from_f(o, o_dt, ob + i, load_as_f(o, o_dt, ob + i) * s);
    }
}

__global__ void xielu_kernel(const void* __restrict__ x, int dt, float ap, float an, void* __restrict__ out, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    store_from_f(out, dt, i, xielu(load_as_f(x, dt, i), ap, an));
}

}  // namespace

static size_t norm_smem(int H) { return ((size_t)H + NORM_WARPS) * sizeof(float); }

// A row is held in shared memory as float32: rows beyond 48 KB need the kernel's limit raised, rows beyond what an SM
// has are refused.
// Eight columns at a time: rows and groups of whole eights, every base on 16 bytes (null pointers pass).
static bool eights(int H, int groups, std::initializer_list<const void*> ps) {
    if (H % 8 || groups < 1 || (H / groups) % 8) return false;
    for (const void* p : ps)
        if (((uintptr_t)p & 15) != 0) return false;
    return true;
}

template <typename K>
static bool row_fits(K kernel, int H) {
    const size_t need = norm_smem(H);
    if (need <= 48 * 1024) return true;
    if (need > 227 * 1024) return false;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need) == cudaSuccess;
}

QNN_API int qnn_group_rmsnorm(const void* x, int x_dt, const void* w, int w_dt, float eps, int groups, void* out,
                              int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (groups < 1 || H % groups) return QNN_ERR_ARGUMENT;
    auto kern = eights(H, groups, {x, w, out}) ? group_rmsnorm_kernel<true> : group_rmsnorm_kernel<false>;
    if (!row_fits(kern, H)) return QNN_ERR_UNSUPPORTED;
    launch_pdl(kern, dim3(T), dim3(NORM_THREADS), norm_smem(H), st, x, x_dt, w, w_dt, eps, groups, out, out_dt, H);
    QNN_LAUNCH_CHECK();
}

// resid: float32 [T, H], updated in place.  a, b: [T, H] or null.  out: null for the add alone.
QNN_API int qnn_add2_group_rmsnorm(float* resid, const void* a, int a_dt, const void* b, int b_dt, const void* w, int w_dt,
                                   float eps, int groups, void* out, int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (out != nullptr && (groups < 1 || H % groups || w == nullptr)) return QNN_ERR_ARGUMENT;
    if (groups < 1) groups = 1;
    auto kern = eights(H, out != nullptr ? groups : 1, {resid, a, b, w, out}) ? add2_group_rmsnorm_kernel<true>
                                                                             : add2_group_rmsnorm_kernel<false>;
    if (!row_fits(kern, H)) return QNN_ERR_UNSUPPORTED;
    launch_pdl(kern, dim3(T), dim3(NORM_THREADS), norm_smem(H), st, resid, a, a_dt, b, b_dt, w, w_dt, eps, groups, out, out_dt,
               H);
    QNN_LAUNCH_CHECK();
}

// pos_table: [n_pos, H]; a position outside it adds nothing (the engine admits none).  normed: null for the rows alone.
QNN_API int qnn_embed_pos(const int* tokens, const void* table, int t_dt, float scale, const void* pos_table, int p_dt,
                          const int* tok_pos, int n_pos, float* out, const void* w, int w_dt, float eps, int groups,
                          void* normed, int n_dt, int T, int H, int V, cudaStream_t st) {
    if (T <= 0) return 0;
    if (normed != nullptr && (groups < 1 || H % groups || w == nullptr)) return QNN_ERR_ARGUMENT;
    if (groups < 1) groups = 1;
    auto kern = eights(H, normed != nullptr ? groups : 1, {table, pos_table, out, w, normed}) ? embed_pos_kernel<true>
                                                                                               : embed_pos_kernel<false>;
    if (!row_fits(kern, H)) return QNN_ERR_UNSUPPORTED;
    launch_pdl(kern, dim3(T), dim3(NORM_THREADS), norm_smem(H), st, tokens, table, t_dt, scale, pos_table, p_dt, tok_pos, n_pos,
               out, w, w_dt, eps, groups, normed, n_dt, H, V);
    QNN_LAUNCH_CHECK();
}

// o: [T, ldo] rows of which the first N columns are gated in place; g: [T, ldg] rows, the gate's logits in their
// first N columns.  float32 rows take the accurate exponential.
QNN_API int qnn_sigmoid_gate(void* o, int o_dt, long long ldo, const void* g, int g_dt, long long ldg, int T, int N,
                             cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (ldo < N || ldg < N) return QNN_ERR_ARGUMENT;
    const bool vec = N % 8 == 0 && ldo % 8 == 0 && ldg % 8 == 0 && (((uintptr_t)o | (uintptr_t)g) & 15) == 0;
    const int threads = N >= (vec ? 2048 : 1024) ? 256 : 128;
    launch_pdl(vec ? sigmoid_gate_kernel<true> : sigmoid_gate_kernel<false>, dim3(T), dim3(threads), 0, st, o, o_dt, ldo, g,
               g_dt, ldg, N, (int)(o_dt == QNN_DT_F32 && g_dt == QNN_DT_F32));
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_xielu(const void* x, int dt, float ap, float an, void* out, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    launch_pdl(xielu_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, dt, ap, an, out, (size_t)n);
    QNN_LAUNCH_CHECK();
}
