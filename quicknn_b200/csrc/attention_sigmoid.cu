// Attention whose weights are sigmoids, not a softmax, and whose heads talk to each other:
//
//   s_g(i, j) = scale q_g(i) . k_c(g)(j) + pb_g              c(g): the key/value head of query head g
//   w_g(i, j) = sigmoid(s_g(i, j))  for the keys j that i sees, 0 otherwise; nothing is normalised over j
//   m_h(i, j) = sum_g talk[h, g] w_g(i, j)                   the heads' weights mixed by a matrix [H, H]
//   o_h(i)    = gate_h(i) * sum_j m_h(i, j) v_c(h)(j)        gate_h(i) = sigmoid(a logit per token and head)
//
// What a position sees is a parameter (`mask_kind`, `mask_size`): every earlier position; the last `size` positions (a
// sliding window); or the earlier positions of its own chunk of `size` positions, chunks counted from position 0 of
// the sequence (position i sees j <= i with floor(i / size) == floor(j / size)).
//
//   qnn_sigattn         one kernel for whole prompts, for steps that continue sequences and for single tokens: a key
//                       at or after the position of the step's first row of the sequence is read from the step's
//                       packed q | k | v rows (`own_rows`), an earlier one from the paged cache line (ring aware); with
//                       own_rows = 0 every key comes from the cache (a decode step, after its append).
//   qnn_sigattn_finish  sums the partial outputs of the key ranges in order and applies the gate (only with ranges)
//
// A block per (token, key range) holds the token's queries of all heads in shared memory as float32 and walks its
// keys in tiles: scores and sigmoids of all heads for the tile, the mix over heads, then the weighted sum of the
// values.  Because nothing is normalised the tiles, and the key ranges of a long context, simply add up.  Scores,
// weights, the mix and the sums are float32 in both precisions; the order of every sum depends on the sizes and on
// the token's own position only, never on the batch.
#include "common.cuh"

using namespace qnn;

#define QNN_MASK_CAUSAL 0
#define QNN_MASK_WINDOW 1
#define QNN_MASK_CHUNK 2

namespace {

constexpr int SA_THREADS = 256;
constexpr int SA_NACC = 16;                         // outputs per thread: heads * head size up to 4096

template <typename T> struct SaPad { static constexpr int N = 1; };
template <> struct SaPad<bf16> { static constexpr int N = 2; };      // rows of the tiles an odd number of words apart

template <typename T, int KT, bool VEC>
__global__ void __launch_bounds__(SA_THREADS)
sigattn_kernel(const T* __restrict__ qkv, long long ld, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
               const int* __restrict__ page_table, int max_pages, int page_size, int ring,
               const int* __restrict__ tok_pos, const int* __restrict__ tok_row0, const int* __restrict__ tok_slot,
               int own_rows, int mask_kind, int mask_size, float scale, const float* __restrict__ pb,
               const float* __restrict__ talk, const void* __restrict__ gate, int g_dt, long long ldg,
               T* __restrict__ out, long long ldo, float* __restrict__ partial, int n_tokens, int H, int G, int D) {
    extern __shared__ __align__(16) float sm[];
    const int HD = H * D, GD = G * D, pitch = GD + SaPad<T>::N, per = H / G;
    float* qs = sm;                                  // [H * D] queries times the scale
    float* ws = qs + HD;                             // [H][KT] weights of the tile
    float* wm = ws + H * KT;                         // [H][KT] mixed over heads
    float* tk = wm + H * KT;                         // [H][H]
    float* pbs = tk + H * H;                         // [H]
    T* ks = reinterpret_cast<T*>(pbs + H + (H & 1)); // [KT][pitch]
    T* vs = ks + (size_t)KT * pitch;
    pdl_wait();
    const int t = blockIdx.x, split = blockIdx.y, n_split = gridDim.y;
    const int tid = threadIdx.x;
    const int slot = tok_slot != nullptr ? tok_slot[t] : 0;
    const int pos = tok_pos[t];
    float acc[SA_NACC];
#pragma unroll
    for (int a = 0; a < SA_NACC; ++a) acc[a] = 0.f;
    if (slot >= 0) {
        int lo = 0;
        if (mask_kind == QNN_MASK_WINDOW) lo = max(0, pos - mask_size + 1);
        else if (mask_kind == QNN_MASK_CHUNK) lo = (pos / mask_size) * mask_size;
        const int row0 = own_rows ? tok_row0[t] : 0;
        const int pos0 = own_rows ? tok_pos[row0] : pos + 1;          // keys from here on are rows of this step
        for (int i = tid; i < HD; i += SA_THREADS) qs[i] = to_f(qkv[(size_t)t * ld + i]) * scale;
        for (int i = tid; i < H * H; i += SA_THREADS) tk[i] = talk != nullptr ? talk[i] : ((i / H) == (i % H) ? 1.f : 0.f);
        for (int i = tid; i < H; i += SA_THREADS) pbs[i] = pb != nullptr ? pb[i] : 0.f;
        const int n_tiles = (pos - lo) / KT + 1;
        constexpr int V = VEC ? Vec16<T>::N : 1;
        const int chunks = GD / V;
        for (int kt = split; kt < n_tiles; kt += n_split) {
            const int j0 = lo + kt * KT, nk = min(KT, pos + 1 - j0);
            __syncthreads();
            for (int idx = tid; idx < KT * chunks; idx += SA_THREADS) {
                const int j = idx / chunks, c = (idx - j * chunks) * V;
                float kv[V], vv[V];
#pragma unroll
                for (int e = 0; e < V; ++e) kv[e] = vv[e] = 0.f;
                if (j < nk) {
                    const int p = j0 + j;
                    const T *kp, *vp;
                    if (p >= pos0) {
                        kp = qkv + (size_t)(row0 + p - pos0) * ld + HD + c;
                        vp = kp + GD;
                    } else {
                        const int r = ring > 0 ? p % ring : p;
                        const int page = page_table[(size_t)slot * max_pages + r / page_size];
                        const size_t at = (((size_t)page * G + c / D) * page_size + (r % page_size)) * D + (c % D);
                        kp = k_pool + at;
                        vp = v_pool + at;
                    }
                    if (VEC) {
                        Vec16<T> a, b;
                        a.load(kp);
                        b.load(vp);
                        a.unpack(kv);
                        b.unpack(vv);
                    } else {
                        kv[0] = to_f(*kp);
                        vv[0] = to_f(*vp);
                    }
                }
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    ks[(size_t)j * pitch + c + e] = from_f<T>(kv[e]);
                    vs[(size_t)j * pitch + c + e] = from_f<T>(vv[e]);
                }
            }
            __syncthreads();
            for (int idx = tid; idx < H * KT; idx += SA_THREADS) {
                const int g = idx / KT, j = idx - g * KT;
                float w = 0.f;
                if (j < nk) {
                    const float* qg = qs + g * D;
                    const T* kj = ks + (size_t)j * pitch + (g / per) * D;
                    float s = 0.f;
                    for (int d = 0; d < D; ++d) s += qg[d] * to_f(kj[d]);
                    w = 1.f / (1.f + expf(-(s + pbs[g])));
                }
                ws[idx] = w;
            }
            __syncthreads();
            for (int idx = tid; idx < H * KT; idx += SA_THREADS) {
                const int h = idx / KT, j = idx - h * KT;
                float m = 0.f;
                for (int g = 0; g < H; ++g) m += tk[h * H + g] * ws[g * KT + j];
                wm[idx] = m;
            }
            __syncthreads();
#pragma unroll
            for (int a = 0; a < SA_NACC; ++a) {
                const int idx = tid + a * SA_THREADS;
                if (idx < HD) {
                    const int h = idx / D, d = idx - h * D;
                    const float* mh = wm + h * KT;
                    const T* vc = vs + (h / per) * D + d;
                    float s = acc[a];
#pragma unroll 8
                    for (int j = 0; j < KT; ++j) s += mh[j] * to_f(vc[(size_t)j * pitch]);
                    acc[a] = s;
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < SA_NACC; ++a) {
        const int idx = tid + a * SA_THREADS;
        if (idx < HD) {
            if (n_split > 1) {
                partial[((size_t)split * n_tokens + t) * HD + idx] = acc[a];
            } else {
                float v = acc[a];
                if (gate != nullptr) v *= 1.f / (1.f + expf(-load_as_f(gate, g_dt, (size_t)t * ldg + idx / D)));
                out[(size_t)t * ldo + idx] = from_f<T>(v);
            }
        }
    }
}

template <typename T>
__global__ void sigattn_finish_kernel(const float* __restrict__ partial, int n_split, const void* __restrict__ gate,
                                      int g_dt, long long ldg, T* __restrict__ out, long long ldo, int n_tokens, int HD,
                                      int D) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_tokens * HD) return;
    const size_t t = i / HD;
    const int idx = (int)(i - t * HD);
    float v = 0.f;
    for (int s = 0; s < n_split; ++s) v += partial[((size_t)s * n_tokens + t) * HD + idx];
    if (gate != nullptr) v *= 1.f / (1.f + expf(-load_as_f(gate, g_dt, t * ldg + idx / D)));
    out[t * ldo + idx] = from_f<T>(v);
}

size_t sa_smem(int H, int G, int D, int KT, size_t elem) {
    const size_t pitch = (size_t)G * D + (elem == 2 ? 2 : 1);
    return ((size_t)H * D + 2 * (size_t)H * KT + (size_t)H * H + H + (H & 1)) * sizeof(float) + 2 * (size_t)KT * pitch * elem;
}

template <typename T, int KT, bool VEC>
int sa_launch(dim3 grid, size_t smem, cudaStream_t st, const void* qkv, long long ld, const void* k_pool, const void* v_pool,
              const int* page_table, int max_pages, int page_size, int ring, const int* tok_pos, const int* tok_row0,
              const int* tok_slot, int own_rows, int mask_kind, int mask_size, float scale, const float* pb,
              const float* talk, const void* gate, int g_dt, long long ldg, void* out, long long ldo, float* partial,
              int n_tokens, int H, int G, int D) {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        const cudaError_t rc = cudaFuncSetAttribute(sigattn_kernel<T, KT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    (int)smem);
        if (rc != cudaSuccess) return (int)rc;
        allowed = smem;
    }
    launch_pdl(sigattn_kernel<T, KT, VEC>, grid, dim3(SA_THREADS), smem, st, (const T*)qkv, ld, (const T*)k_pool,
               (const T*)v_pool, page_table, max_pages, page_size, ring, tok_pos, tok_row0, tok_slot, own_rows, mask_kind,
               mask_size, scale, pb, talk, gate, g_dt, ldg, (T*)out, ldo, partial, n_tokens, H, G, D);
    QNN_LAUNCH_CHECK();
}

}  // namespace

// Sizes that the kernel takes: heads * head size up to 4096, kv heads that divide the heads, and tiles of at least 8 keys
// within 200 KB of shared memory.  Returns 1 or 0; no launch.
QNN_API int qnn_sigattn_supports(int dtype, int H, int G, int D) {
    if (H <= 0 || G <= 0 || D <= 0 || H % G || (long long)H * D > SA_THREADS * SA_NACC) return 0;
    return sa_smem(H, G, D, 8, dtype == QNN_DT_BF16 ? 2 : 4) <= 200 * 1024 ? 1 : 0;
}

// qkv: [T, ld] rows of `dtype`: H query heads, G key heads, G value heads of D columns.  k_pool / v_pool:
// [pages][G][page_size][D] of the same type (may be null when every key is a row of the step); page_table:
// [slots, max_pages].  tok_pos / tok_row0 / tok_slot: per row its position, the first row of its sequence in this step,
// and its slot (negative: a row of no sequence, whose output is zero).  pb: [H] float32 or null; talk: [H, H] float32 or
// null (no mixing); gate: logits [T, ldg] of `g_dt`, one per head, or null.  out: [T, ldo] of `dtype`.  n_split > 1:
// the keys of a token are walked by that many blocks, `partial` is float32 [n_split, T, H * D].
QNN_API int qnn_sigattn(const void* qkv, int dtype, long long ld, const void* k_pool, const void* v_pool,
                        const int* page_table, int max_pages, int page_size, int ring, const int* tok_pos,
                        const int* tok_row0, const int* tok_slot, int own_rows, int mask_kind, int mask_size, float scale,
                        const float* pb, const float* talk, const void* gate, int g_dt, long long ldg, void* out,
                        long long ldo, float* partial, int n_split, int T, int H, int G, int D, cudaStream_t st) {
    if (T <= 0) return 0;
    if (!qnn_sigattn_supports(dtype, H, G, D)) return QNN_ERR_UNSUPPORTED;
    if (mask_kind < 0 || mask_kind > 2 || (mask_kind != QNN_MASK_CAUSAL && mask_size < 1) || n_split < 1 || n_split > 65535)
        return QNN_ERR_ARGUMENT;
    if (tok_pos == nullptr || (own_rows && tok_row0 == nullptr) || (n_split > 1 && partial == nullptr)) return QNN_ERR_ARGUMENT;
    if (!own_rows && (k_pool == nullptr || v_pool == nullptr || page_table == nullptr)) return QNN_ERR_ARGUMENT;
    const size_t elem = dtype == QNN_DT_BF16 ? 2 : 4;
    int KT = 32;
    while (KT > 8 && sa_smem(H, G, D, KT, elem) > 200 * 1024) KT /= 2;
    const size_t smem = sa_smem(H, G, D, KT, elem);
    const bool vec = (D * elem) % 16 == 0 && (ld * elem) % 16 == 0 && ((uintptr_t)qkv % 16) == 0 &&
                     ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0;
    const dim3 grid(T, n_split);
    int rc;
#define QNN_SA(TT, KTV)                                                                                               \
    rc = vec ? sa_launch<TT, KTV, true>(grid, smem, st, qkv, ld, k_pool, v_pool, page_table, max_pages, page_size, ring,  \
                                        tok_pos, tok_row0, tok_slot, own_rows, mask_kind, mask_size, scale, pb, talk,     \
                                        gate, g_dt, ldg, out, ldo, partial, T, H, G, D)                                   \
             : sa_launch<TT, KTV, false>(grid, smem, st, qkv, ld, k_pool, v_pool, page_table, max_pages, page_size, ring, \
                                         tok_pos, tok_row0, tok_slot, own_rows, mask_kind, mask_size, scale, pb, talk,    \
                                         gate, g_dt, ldg, out, ldo, partial, T, H, G, D)
    if (dtype == QNN_DT_BF16) {
        if (KT == 32) QNN_SA(bf16, 32); else if (KT == 16) QNN_SA(bf16, 16); else QNN_SA(bf16, 8);
    } else {
        if (KT == 32) QNN_SA(float, 32); else if (KT == 16) QNN_SA(float, 16); else QNN_SA(float, 8);
    }
#undef QNN_SA
    if (rc != 0 || n_split == 1) return rc;
    const size_t n = (size_t)T * H * D;
    if (dtype == QNN_DT_BF16)
        launch_pdl(sigattn_finish_kernel<bf16>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const float*)partial,
                   n_split, gate, g_dt, ldg, (bf16*)out, ldo, T, H * D, D);
    else
        launch_pdl(sigattn_finish_kernel<float>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const float*)partial,
                   n_split, gate, g_dt, ldg, (float*)out, ldo, T, H * D, D);
    QNN_LAUNCH_CHECK();
}
