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
//   qnn_sigattn_prefill_mma   whole prompts in bfloat16 on the tensor cores (further down)
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

__device__ __forceinline__ void sa_cp_async_16(unsigned smem_dst, const void* gmem_src, bool valid) {
    const int bytes = valid ? 16 : 0;                // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_dst), "l"(gmem_src), "r"(bytes));
}
__device__ __forceinline__ void sa_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 0;\n" ::);
}

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
    // bfloat16 rows in whole 16-byte pieces: keys and values are read from shared memory two at a time
    constexpr bool PAIR = VEC && sizeof(T) == 2;
    // VEC: rows of the tiles start on 16 bytes (they are filled by cp.async); else rows an odd number of words apart
    const int HD = H * D, GD = G * D, pitch = GD + (VEC ? (int)(16 / sizeof(T)) : SaPad<T>::N), per = H / G;
    float* qs = sm;                                  // [H * D] queries times the scale
    float* ws = qs + HD;                             // [H][KT] weights of the tile
    float* wm = ws + H * KT;                         // [H][KT] mixed over heads
    float* tk = wm + H * KT;                         // [H][H]
    float* pbs = tk + H * H;                         // [H]
    T* ks = reinterpret_cast<T*>(sm + ((HD + 2 * H * KT + H * H + H + 3) & ~3));   // [KT][pitch], on 16 bytes
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
            if (VEC) {
                // a warp per key row: the row's place is worked out once, its pieces go global -> shared by cp.async
                const int warp = tid >> 5, lane = tid & 31;
                const unsigned sk = (unsigned)__cvta_generic_to_shared(ks), sv = (unsigned)__cvta_generic_to_shared(vs);
                constexpr int PIECE = 16 / sizeof(T);
                for (int j = warp; j < KT; j += SA_THREADS / 32) {
                    const bool valid = j < nk;
                    const int p = j0 + j;
                    const T *kp = qkv, *vp = qkv;
                    size_t head_step = D;             // from one key/value head's columns to the next's
                    if (valid && p >= pos0) {
                        kp = qkv + (size_t)(row0 + p - pos0) * ld + HD;
                        vp = kp + GD;
                    } else if (valid) {
                        const int r = ring > 0 ? p % ring : p;
                        const int page = page_table[(size_t)slot * max_pages + r / page_size];
                        const size_t at = ((size_t)page * G * page_size + (r % page_size)) * D;
                        kp = k_pool + at;
                        vp = v_pool + at;
                        head_step = (size_t)page_size * D;
                    }
                    for (int c = 0; c < G; ++c)
                        for (int d = lane * PIECE; d < D; d += 32 * PIECE) {
                            const unsigned dst = (unsigned)(((size_t)j * pitch + c * D + d) * sizeof(T));
                            sa_cp_async_16(sk + dst, kp + c * head_step + d, valid);
                            sa_cp_async_16(sv + dst, vp + c * head_step + d, valid);
                        }
                }
                sa_cp_async_wait_all();
            } else
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
                        if (PAIR) {                  // the 16 bytes as they came, four words (rows are whole words apart)
                            const uint32_t* aw = reinterpret_cast<const uint32_t*>(&a.raw);
                            const uint32_t* bw = reinterpret_cast<const uint32_t*>(&b.raw);
                            uint32_t* kd = reinterpret_cast<uint32_t*>(ks + (size_t)j * pitch + c);
                            uint32_t* vd = reinterpret_cast<uint32_t*>(vs + (size_t)j * pitch + c);
#pragma unroll
                            for (int e = 0; e < 4; ++e) { kd[e] = aw[e]; vd[e] = bw[e]; }
                            continue;
                        }
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
            if (VEC) {
                // a lane per score, as below; rows start on 16 bytes here, so lane j begins its walk along the head
                // (j / 8) pairs further on and wraps: the 32 lanes of a key tile then read 32 different banks
                for (int idx = tid; idx < H * KT; idx += SA_THREADS) {
                    const int g = idx / KT, j = idx - g * KT;
                    float w = 0.f;
                    if (j < nk) {
                        const float2* q2 = reinterpret_cast<const float2*>(qs + g * D);
                        const T* kj = ks + (size_t)j * pitch + (g / per) * D;
                        const int half = D / 2;
                        int e = (j >> 3) & 3;
                        if (e >= half) e = 0;
                        float sc = 0.f;
                        for (int n = 0; n < half; ++n) {
                            float2 kf;
                            if (sizeof(T) == 2) kf = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(kj)[e]);
                            else kf = reinterpret_cast<const float2*>(kj)[e];
                            const float2 qf = q2[e];
                            sc = fmaf(qf.x, kf.x, sc);
                            sc = fmaf(qf.y, kf.y, sc);
                            if (++e == half) e = 0;
                        }
                        w = 1.f / (1.f + expf(-(sc + pbs[g])));
                    }
                    ws[idx] = w;
                }
            } else
            for (int idx = tid; idx < H * KT; idx += SA_THREADS) {
                const int g = idx / KT, j = idx - g * KT;
                float w = 0.f;
                if (j < nk) {
                    const float* qg = qs + g * D;
                    const T* kj = ks + (size_t)j * pitch + (g / per) * D;
                    float s = 0.f;
                    if (PAIR) {
                        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(kj);
                        const float2* q2 = reinterpret_cast<const float2*>(qg);
#pragma unroll 4
                        for (int d = 0; d < D / 2; ++d) {
                            const float2 kf = __bfloat1622float2(k2[d]), qf = q2[d];
                            s = fmaf(qf.x, kf.x, s);
                            s = fmaf(qf.y, kf.y, s);
                        }
                    } else {
                        for (int d = 0; d < D; ++d) s += qg[d] * to_f(kj[d]);
                    }
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
            if (PAIR) {                              // accumulators 2a and 2a + 1: columns 2 idx and 2 idx + 1
#pragma unroll
                for (int a = 0; a < SA_NACC / 2; ++a) {
                    const int idx = 2 * (tid + a * SA_THREADS);
                    if (idx < HD) {
                        const int h = idx / D, d = idx - h * D;
                        const float* mh = wm + h * KT;
                        const T* vc = vs + (h / per) * D + d;
                        float s0 = acc[2 * a], s1 = acc[2 * a + 1];
#pragma unroll 8
                        for (int j = 0; j < KT; ++j) {
                            const float2 vf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vc + (size_t)j * pitch));
                            s0 = fmaf(mh[j], vf.x, s0);
                            s1 = fmaf(mh[j], vf.y, s1);
                        }
                        acc[2 * a] = s0;
                        acc[2 * a + 1] = s1;
                    }
                }
            } else {
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
    }
#pragma unroll
    for (int a = 0; a < SA_NACC; ++a) {
        const int idx = PAIR ? 2 * (tid + (a >> 1) * SA_THREADS) + (a & 1) : tid + a * SA_THREADS;
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

size_t sa_smem(int H, int G, int D, int KT, size_t elem, bool vec = true) {
    const size_t pitch = (size_t)G * D + (vec ? 16 / elem : (elem == 2 ? 2 : 1));        // the wider of the two when asked in general
    const size_t floats = ((size_t)H * D + 2 * (size_t)H * KT + (size_t)H * H + H + 3) & ~(size_t)3;
    return floats * sizeof(float) + 2 * (size_t)KT * pitch * elem;
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


// ---- whole prompts on the tensor cores (bfloat16) -------------------------------------------------------------------
// A block owns 16 query rows of one sequence and all heads, a warp per query head.  Per tile of KT keys: every warp
// forms its head's scores S = Q_g K^T (mma.sync m16n8k16, Q, K and V fragments by ldmatrix from padded rows), the
// sigmoids in float32, and leaves them in shared memory; after a barrier every warp mixes the heads' weights for its
// own head h from there, in float32 and straight into the A operand of O_h += M_h V (the mix needs every head's weight
// of an element, which is why one block holds all heads of its rows and why the weights pass through shared
// memory).  Keys and values are read from the step's packed rows.  The mixed weights are rounded to bfloat16 for the
// product with the values, as the softmax kernels round theirs; sums are float32.

__device__ __forceinline__ void sa_ldmatrix_x4(uint32_t (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sa_ldmatrix_x4_trans(uint32_t (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sa_mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sa_pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

constexpr int SAM_ROWS = 16;          // query rows of a block

// Keys and values of a tile are loaded (cp.async) into one of `stages` buffers while the tile before is worked on.
// `tiles_per_range` > 0: the key tiles of a query tile are cut into ranges of that many, a block (blockIdx.z) each; the
// blocks leave float32 partial outputs in `partial` [ranges][rows][H * D] (zeros where a range holds no tile of the
// query tile), which qnn_sigattn_finish's kernel sums in order: nothing is normalised over the keys, so ranges add up.
template <int D, int KT>
__global__ void __launch_bounds__(D > 128 ? 256 : 512)
sigattn_prefill_mma_kernel(const bf16* __restrict__ qkv, long long ld, const int* __restrict__ seq_row0,
                           const int* __restrict__ seq_len, int mask_kind, int mask_size, float scale,
                           const float* __restrict__ pb, const float* __restrict__ talk, const void* __restrict__ gate,
                           int g_dt, long long ldg, bf16* __restrict__ out, long long ldo, int H, int G, int stages,
                           int tiles_per_range, float* __restrict__ partial, int n_rows) {
    extern __shared__ __align__(16) unsigned char sa_smem_raw[];
    constexpr int WP = KT + 8;                       // pitch of a row of weights, floats
    const int HD = H * D, GD = G * D, per = H / G;
    const int QP = HD + 8, KP = GD + 8;              // pitches in elements: rows 16 bytes apart in the banks
    bf16* qs = reinterpret_cast<bf16*>(sa_smem_raw);                 // [16][QP]
    bf16* kv = qs + (size_t)SAM_ROWS * QP;                           // [stages][keys | values][KT][KP]
    float* ws = reinterpret_cast<float*>(kv + (size_t)stages * 2 * KT * KP);      // [H][16][WP]
    float* tk = ws + (size_t)H * SAM_ROWS * WP;                      // [H][H]
    pdl_wait();
    const int b = blockIdx.y, len = seq_len[b];
    const int ntiles = (len + SAM_ROWS - 1) / SAM_ROWS;
    if ((int)blockIdx.x >= ntiles) return;
    const int tile = ntiles - 1 - blockIdx.x;        // the longest rows first
    const int r0 = tile * SAM_ROWS, row0 = seq_row0[b];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g_ = lane >> 2, t_ = lane & 3, nthr = blockDim.x;
    const int h = warp;                              // this warp's query head, and the head it mixes for
    const int c = h / per;                           // its key/value head
    const unsigned sQ = (unsigned)__cvta_generic_to_shared(qs), sKV = (unsigned)__cvta_generic_to_shared(kv);
    const unsigned stage_bytes = (unsigned)(2 * KT * KP) * 2, v_off = (unsigned)(KT * KP) * 2;
    const int last = min(r0 + SAM_ROWS, len) - 1;    // the last position of the tile
    int lo = 0;                                      // the first key that any row of the tile sees
    if (mask_kind == QNN_MASK_WINDOW) lo = max(0, r0 - mask_size + 1);
    else if (mask_kind == QNN_MASK_CHUNK) lo = (r0 / mask_size) * mask_size;
    const int all_tiles = (last - lo) / KT + 1;
    const int kt0 = tiles_per_range > 0 ? (int)blockIdx.z * tiles_per_range : 0;
    const int kt1 = tiles_per_range > 0 ? min(all_tiles, kt0 + tiles_per_range) : all_tiles;
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    auto load_kv = [&](int kt, int stage) {
        const int j0 = lo + kt * KT, chunks = GD / 8;
        const unsigned dst = sKV + stage * stage_bytes;
        for (int idx = tid; idx < KT * chunks; idx += nthr) {
            const int row = idx / chunks, ch = idx - row * chunks;
            const bool valid = j0 + row <= last;
            const bf16* src = qkv + (size_t)(row0 + (valid ? j0 + row : 0)) * ld + HD + ch * 8;
            sa_cp_async_16(dst + (unsigned)(row * KP + ch * 8) * 2, src, valid);
            sa_cp_async_16(dst + v_off + (unsigned)(row * KP + ch * 8) * 2, src + GD, valid);
        }
    };
    if (kt0 < kt1) {
        for (int i = tid; i < H * H; i += nthr) tk[i] = talk != nullptr ? talk[i] : ((i / H) == (i % H) ? 1.f : 0.f);
        const int chunks = HD / 8;
        for (int idx = tid; idx < SAM_ROWS * chunks; idx += nthr) {
            const int row = idx / chunks, ch = idx - row * chunks;
            const bool valid = r0 + row < len;
            sa_cp_async_16(sQ + (unsigned)(row * QP + ch * 8) * 2, qkv + (size_t)(row0 + (valid ? r0 + row : 0)) * ld + ch * 8, valid);
        }
        load_kv(kt0, 0);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    const float bias = pb != nullptr ? pb[h] : 0.f;
    for (int kt = kt0; kt < kt1; ++kt) {
        const int j0 = lo + kt * KT;
        const int stage = stages > 1 ? ((kt - kt0) & 1) : 0;
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();                             // this tile has come; the tile before is read, its weights too
        if (stages > 1 && kt + 1 < kt1) {
            load_kv(kt + 1, stage ^ 1);
            asm volatile("cp.async.commit_group;\n" ::);
        }
        const unsigned sK = sKV + stage * stage_bytes, sV = sK + v_off;
        // the scores of this warp's head
        float s[KT / 8][4];
#pragma unroll
        for (int i = 0; i < KT / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {
            uint32_t a[4];
            sa_ldmatrix_x4(a, sQ + (unsigned)((lane & 15) * QP + h * D + k16 * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int np = 0; np < KT / 16; ++np) {
                uint32_t bfr[4];
                const int row = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                sa_ldmatrix_x4(bfr, sK + (unsigned)(row * KP + c * D + k16 * 16 + ((lane >> 3) & 1) * 8) * 2);
                sa_mma_16816(s[np * 2], a, bfr[0], bfr[1]);
                sa_mma_16816(s[np * 2 + 1], a, bfr[2], bfr[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = g_ + half * 8, i = r0 + row;
                int first = 0;
                if (mask_kind == QNN_MASK_WINDOW) first = i - mask_size + 1;
                else if (mask_kind == QNN_MASK_CHUNK) first = (i / mask_size) * mask_size;
                float w2[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = j0 + nt * 8 + 2 * t_ + e;
                    const bool seen = j <= i && j >= first && i < len;
                    w2[e] = seen ? __fdividef(1.f, 1.f + __expf(-(s[nt][half * 2 + e] * scale + bias))) : 0.f;
                }
                *reinterpret_cast<float2*>(ws + ((size_t)h * SAM_ROWS + row) * WP + nt * 8 + 2 * t_) = make_float2(w2[0], w2[1]);
            }
        __syncthreads();
        // this head's mix of all heads' weights, as the A operand; O += M V
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            float m[4][2];
#pragma unroll
            for (int q = 0; q < 4; ++q) m[q][0] = m[q][1] = 0.f;
            for (int g = 0; g < H; ++g) {
                const float tg = tk[h * H + g];
                const float* wg = ws + (size_t)g * SAM_ROWS * WP + kk * 16 + 2 * t_;
                const float2 x0 = *reinterpret_cast<const float2*>(wg + (size_t)g_ * WP);
                const float2 x1 = *reinterpret_cast<const float2*>(wg + (size_t)(g_ + 8) * WP);
                const float2 x2 = *reinterpret_cast<const float2*>(wg + (size_t)g_ * WP + 8);
                const float2 x3 = *reinterpret_cast<const float2*>(wg + (size_t)(g_ + 8) * WP + 8);
                m[0][0] += tg * x0.x; m[0][1] += tg * x0.y;
                m[1][0] += tg * x1.x; m[1][1] += tg * x1.y;
                m[2][0] += tg * x2.x; m[2][1] += tg * x2.y;
                m[3][0] += tg * x3.x; m[3][1] += tg * x3.y;
            }
            uint32_t a[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) a[q] = sa_pack_bf16(m[q][0], m[q][1]);
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                uint32_t bfr[4];
                const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                sa_ldmatrix_x4_trans(bfr, sV + (unsigned)(row * KP + c * D + dp * 16 + (lane >> 4) * 8) * 2);
                sa_mma_16816(o[dp * 2], a, bfr[0], bfr[1]);
                sa_mma_16816(o[dp * 2 + 1], a, bfr[2], bfr[3]);
            }
        }
        if (stages == 1 && kt + 1 < kt1) {
            __syncthreads();                         // the one buffer is read before it is filled again
            load_kv(kt + 1, 0);
            asm volatile("cp.async.commit_group;\n" ::);
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int i = r0 + g_ + half * 8;
        if (i >= len) continue;
        const size_t t = (size_t)(row0 + i);
        if (tiles_per_range > 0) {
            float* dst = partial + ((size_t)blockIdx.z * n_rows + t) * HD + h * D + 2 * t_;
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd)
                *reinterpret_cast<float2*>(dst + nd * 8) = make_float2(o[nd][half * 2], o[nd][half * 2 + 1]);
            continue;
        }
        float gt = 1.f;
        if (gate != nullptr) gt = 1.f / (1.f + expf(-load_as_f(gate, g_dt, t * ldg + h)));
#pragma unroll
        for (int nd = 0; nd < D / 8; ++nd)
            *reinterpret_cast<uint32_t*>(out + t * ldo + h * D + nd * 8 + 2 * t_) =
                sa_pack_bf16(o[nd][half * 2] * gt, o[nd][half * 2 + 1] * gt);
    }
}

size_t sam_smem(int H, int G, int D, int KT, int stages) {
    return ((size_t)SAM_ROWS * (H * D + 8) + (size_t)stages * 2 * KT * (G * D + 8)) * 2 +
           ((size_t)H * SAM_ROWS * (KT + 8) + (size_t)H * H) * sizeof(float);
}

// Keys per tile: 32 where two blocks of that size fit an SM together or where tiles of 16 would not let two fit either;
// else 16 (two blocks per SM hide each other's barriers and loads).  QNN_SIGATTN_KT=16|32 fixes it, for measurements.
int sam_tile(int H, int G, int D) {
    static int fixed = -1;
    if (fixed < 0) {
        const char* e = getenv("QNN_SIGATTN_KT");
        fixed = e != nullptr ? atoi(e) : 0;
    }
    if (fixed == 16 || fixed == 32) return sam_smem(H, G, D, fixed, 1) <= 220 * 1024 ? fixed : 16;
    const size_t half = 113 * 1024;
    if (sam_smem(H, G, D, 32, 2) <= half) return 32;
    if (sam_smem(H, G, D, 16, 2) <= half) return 16;
    return sam_smem(H, G, D, 32, 2) <= 220 * 1024 ? 32 : 16;
}

template <int D, int KT>
int sam_launch(dim3 grid, int threads, size_t smem, cudaStream_t st, const void* qkv, long long ld, const int* seq_row0,
               const int* seq_len, int mask_kind, int mask_size, float scale, const float* pb, const float* talk,
               const void* gate, int g_dt, long long ldg, void* out, long long ldo, int H, int G, int stages,
               int tiles_per_range, float* partial, int n_rows) {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        const cudaError_t rc = cudaFuncSetAttribute(sigattn_prefill_mma_kernel<D, KT>,
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (rc != cudaSuccess) return (int)rc;
        allowed = smem;
    }
    launch_pdl(sigattn_prefill_mma_kernel<D, KT>, grid, dim3(threads), smem, st, (const bf16*)qkv, ld, seq_row0, seq_len,
               mask_kind, mask_size, scale, pb, talk, gate, g_dt, ldg, (bf16*)out, ldo, H, G, stages, tiles_per_range,
               partial, n_rows);
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
    const bool vec = (D * elem) % 16 == 0 && (ld * elem) % 16 == 0 && ((uintptr_t)qkv % 16) == 0 &&
                     ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0;
    int KT = 32;
    while (KT > 8 && sa_smem(H, G, D, KT, elem, vec) > 200 * 1024) KT /= 2;
    const size_t smem = sa_smem(H, G, D, KT, elem, vec);
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

// Whole prompts (every sequence of the step starts at position 0) in bfloat16 on the tensor cores.  qkv, pb, talk, gate
// and out as for qnn_sigattn; seq_row0 / seq_len: first row and length of each of the B sequences; longest: the longest
// of them; T: rows of the step.  Head sizes 32, 64, 128 (up to 16 heads) and 256 (up to 8 heads), rows in whole 16-byte
// pieces; anything else is refused with QNN_ERR_UNSUPPORTED and the caller takes qnn_sigattn.  Where a query tile sees
// many key tiles they are cut into ranges that run as blocks of their own (qnn_sigattn_prefill_ranges says how many
// for given sizes); `partial` then holds float32 [ranges, T, H * D].
QNN_API int qnn_sigattn_prefill_ranges(int longest, int mask_kind, int mask_size, int H, int G, int D, int* tiles_per_range) {
    const int KT = sam_tile(H, G, D);
    int keys = longest;                              // the most keys that a query tile walks
    if (mask_kind != QNN_MASK_CAUSAL) keys = longest < mask_size + SAM_ROWS ? longest : mask_size + SAM_ROWS;
    const int tiles = (keys + KT - 1) / KT + 1;
    const int per = 512 / KT;                        // a range: 512 keys
    *tiles_per_range = tiles > per + per / 2 ? per : 0;
    return *tiles_per_range > 0 ? (tiles + per - 1) / per : 1;
}

QNN_API int qnn_sigattn_prefill_mma(const void* qkv, long long ld, const int* seq_row0, const int* seq_len, int B,
                                    int longest, int mask_kind, int mask_size, float scale, const float* pb,
                                    const float* talk, const void* gate, int g_dt, long long ldg, void* out,
                                    long long ldo, int H, int G, int D, float* partial, int T, cudaStream_t st) {
    if (B <= 0 || longest <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || H > (D > 128 ? 8 : 16)) return QNN_ERR_UNSUPPORTED;
    if (D != 32 && D != 64 && D != 128 && D != 256) return QNN_ERR_UNSUPPORTED;
    if (ld % 8 || ldo % 2 || ((uintptr_t)qkv % 16) || ((uintptr_t)out % 4) || B > 65535) return QNN_ERR_UNSUPPORTED;
    if (mask_kind < 0 || mask_kind > 2 || (mask_kind != QNN_MASK_CAUSAL && mask_size < 1)) return QNN_ERR_ARGUMENT;
    if (seq_row0 == nullptr || seq_len == nullptr) return QNN_ERR_ARGUMENT;
    int KT = sam_tile(H, G, D), stages = 2;
    if (sam_smem(H, G, D, KT, stages) > 220 * 1024) stages = 1;
    const size_t smem = sam_smem(H, G, D, KT, stages);
    if (smem > 220 * 1024) return QNN_ERR_UNSUPPORTED;
    int tiles_per_range = 0;
    const int ranges = qnn_sigattn_prefill_ranges(longest, mask_kind, mask_size, H, G, D, &tiles_per_range);
    if (ranges > 1 && partial == nullptr) return QNN_ERR_ARGUMENT;
    const dim3 grid((longest + SAM_ROWS - 1) / SAM_ROWS, B, ranges);
    int rc;
#define QNN_SAM(DV)                                                                                                   \
    rc = KT == 32 ? sam_launch<DV, 32>(grid, H * 32, smem, st, qkv, ld, seq_row0, seq_len, mask_kind, mask_size, scale,   \
                                       pb, talk, gate, g_dt, ldg, out, ldo, H, G, stages, tiles_per_range, partial, T)   \
                  : sam_launch<DV, 16>(grid, H * 32, smem, st, qkv, ld, seq_row0, seq_len, mask_kind, mask_size, scale,   \
                                       pb, talk, gate, g_dt, ldg, out, ldo, H, G, stages, tiles_per_range, partial, T)
    if (D == 32) QNN_SAM(32);
    else if (D == 64) QNN_SAM(64);
    else if (D == 128) QNN_SAM(128);
    else QNN_SAM(256);
#undef QNN_SAM
    if (rc != 0 || ranges == 1) return rc;
    const size_t n = (size_t)T * H * D;
    launch_pdl(sigattn_finish_kernel<bf16>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const float*)partial, ranges,
               gate, g_dt, ldg, (bf16*)out, ldo, T, H * D, D);
    QNN_LAUNCH_CHECK();
}
