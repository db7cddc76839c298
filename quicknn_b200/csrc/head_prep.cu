// What happens to the rows of a stacked q | k | v product before attention (or before a recurrence), in one kernel:
//
//   1. a bias over the packed row (optional);
//   2. an RMS norm per head over the first `norm_dim` columns of every query and key head, with a weight per column
//      that all heads share (optional; the heads may be carried wider than norm_dim, with zero columns behind);
//      or, with `norm_whole`, one RMS norm over all query heads together and one over all key heads together (the
//      first norm_dim columns of each head count), with a weight per head and column;
//   3. a rotation of the first `rot` columns of every query and key head by position * inv_freq[j], the pair of
//      frequency j being columns (j, j + rot/2) (half-split) or (2j, 2j + 1) (interleaved);
//   4. the row written back in place, or to another buffer of another element type (float32 rows for a recurrence
//      whose inputs must not be rounded again);
//   5. keys and values appended to a paged cache line (optional; ring aware like qnn_rope_cache_write).
//
// `flags` (QNN_PREP_*): WHOLE = the norm of step 2 over all heads together; NORM_LAST = step 2 comes after step 3 (the
// heads are rotated first and normed then); PLAIN_NORM = the norm has no weights (wq / wk are null); VALUES_ARE_KEYS =
// the source rows hold no value columns: the values are the keys as they are after step 1, before norm and rotation
// (the destination gets them behind the keys, the cache line as its values).
//
// Everything between load and store is float32.  A block per token, a warp per head; the angles of a token are
// formed once per block.  inv_freq comes from the host (float64 arithmetic, rounded once), so any rescaling of the
// frequencies is the caller's business.
#include "common.cuh"

using namespace qnn;

#define QNN_PREP_WHOLE 1
#define QNN_PREP_NORM_LAST 2
#define QNN_PREP_PLAIN_NORM 4
#define QNN_PREP_VALUES_ARE_KEYS 8

namespace {

template <typename T>
__global__ void head_prep_kernel(const T* src, long long lds, void* dst, int dst_dt, long long ldd,
                                 int nq, int nk, int nv, int hd, int norm_dim, int rot, int interleaved,
                                 const void* __restrict__ bias, int b_dt, const void* __restrict__ wq,
                                 const void* __restrict__ wk, int w_dt, float eps, const float* __restrict__ inv_freq,
                                 const int* __restrict__ tok_pos, const int* __restrict__ tok_slot, T* __restrict__ k_pool,
                                 T* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages, int page_size,
                                 int ring, const int* __restrict__ slot_len, int write_cache, int flags) {
    const int norm_whole = flags & QNN_PREP_WHOLE;
    const bool norm_last = flags & QNN_PREP_NORM_LAST, plain = flags & QNN_PREP_PLAIN_NORM;
    const bool v_is_k = flags & QNN_PREP_VALUES_ARE_KEYS;
    extern __shared__ float sm[];                   // [rot/2] (cos, sin) pairs, a head of hd floats per warp, [nq + nk] sums
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos != nullptr ? tok_pos[t] : 0;
    const int slot = tok_slot != nullptr ? tok_slot[t] : -1;
    const int rh = rot / 2;
    float2* angles = reinterpret_cast<float2*>(sm);
    float* heads = sm + 2 * rh;
    for (int j = threadIdx.x; j < rh; j += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        angles[j] = make_float2(cs, sn);
    }
    __syncthreads();
    size_t cache_base = 0;
    bool wr = write_cache && slot >= 0;
    // a prompt longer than the ring keeps only its last `ring` positions (the length after this step is slot_len)
    if (wr && ring > 0 && pos + ring < slot_len[slot]) wr = false;
    if (wr) {
        const int r = ring > 0 ? pos % ring : pos;
        const int page = page_table[(size_t)slot * max_pages + r / page_size];
        cache_base = ((size_t)page * nk * page_size + (r % page_size)) * hd;
    }
    const size_t head_stride = (size_t)page_size * hd;
    const T* row = src + (size_t)t * lds;
    const size_t out_row = (size_t)t * ldd;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    float* mine = heads + (size_t)warp * hd;
    float inv_q = 0.f, inv_k = 0.f;
    if (norm_whole) {
        // every head's sum of squares first, then the heads in order: the same sum whatever the block's size
        float* sums = heads + (size_t)nwarp * hd;
        for (int h = warp; h < nq + nk; h += nwarp) {
            float ss = 0.f;
            for (int c = lane; c < norm_dim; c += 32) {
                float v = to_f(row[(size_t)h * hd + c]);
                if (bias != nullptr) v += load_as_f(bias, b_dt, (size_t)h * hd + c);
                ss += v * v;
            }
            ss = warp_sum(ss);
            if (lane == 0) sums[h] = ss;
        }
        __syncthreads();
        float sq = 0.f, sk = 0.f;
        for (int h = 0; h < nq; ++h) sq += sums[h];
        for (int h = nq; h < nq + nk; ++h) sk += sums[h];
        inv_q = rsqrtf(sq / (float)(nq > 0 ? nq * norm_dim : 1) + eps);
        inv_k = rsqrtf(sk / (float)(nk > 0 ? nk * norm_dim : 1) + eps);
    }
    for (int h = warp; h < nq + nk; h += nwarp) {
        const bool is_k = h >= nq;
        const size_t c0 = (size_t)h * hd;
        float ss = 0.f;
        for (int c = lane; c < hd; c += 32) {
            float v = to_f(row[c0 + c]);
            if (bias != nullptr) v += load_as_f(bias, b_dt, c0 + c);
            mine[c] = v;
            if (c < norm_dim) ss += v * v;
        }
        const void* w = is_k ? wk : wq;
        const bool normed = w != nullptr || (plain && norm_dim > 0);
        if (is_k && v_is_k) {
            // the values are the keys as they stand here: behind the keys in the destination, and the line's values
            T* vc = (wr && v_pool != nullptr) ? v_pool + cache_base + (size_t)(h - nq) * head_stride : nullptr;
            for (int c = lane; c < hd; c += 32) {
                store_from_f(dst, dst_dt, out_row + (size_t)(h + nk) * hd + c, mine[c]);
                if (vc != nullptr) vc[c] = from_f<T>(mine[c]);
            }
        }
        auto norm = [&]() {
            if (norm_last) {                       // the sum of the rotated head's squares
                ss = 0.f;
                for (int c = lane; c < norm_dim; c += 32) ss += mine[c] * mine[c];
            }
            ss = warp_sum(ss);
            const float inv = norm_whole ? (is_k ? inv_k : inv_q) : rsqrtf(ss / (float)norm_dim + eps);
            const size_t w0 = norm_whole ? (size_t)(is_k ? h - nq : h) * norm_dim : 0;
            for (int c = lane; c < norm_dim; c += 32)
                mine[c] = mine[c] * inv * (w != nullptr ? load_as_f(w, w_dt, w0 + c) : 1.f);
        };
        if (normed && !norm_last) norm();
        __syncwarp();
        for (int j = lane; j < rh; j += 32) {
            const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + rh;
            const float a = mine[ia], b = mine[ib];
            const float2 cs = angles[j];
            mine[ia] = a * cs.x - b * cs.y;
            mine[ib] = b * cs.x + a * cs.y;
        }
        __syncwarp();
        if (normed && norm_last) {
            norm();
            __syncwarp();
        }
        T* cache = (is_k && wr) ? k_pool + cache_base + (size_t)(h - nq) * head_stride : nullptr;
        for (int c = lane; c < hd; c += 32) {
            const float v = mine[c];
            store_from_f(dst, dst_dt, out_row + c0 + c, v);
            if (cache != nullptr) cache[c] = from_f<T>(v);
        }
        __syncwarp();
    }
    // values: nv columns behind the keys (nv = kv heads x hd when they go to the cache)
    const size_t v0 = (size_t)(nq + nk) * hd;
    const bool v_cache = wr && v_pool != nullptr;
    if (nv > 0 && !v_is_k && (bias != nullptr || v_cache || (const void*)src != (const void*)dst)) {
        for (int c = threadIdx.x; c < nv; c += blockDim.x) {
            float v = to_f(row[v0 + c]);
            if (bias != nullptr) v += load_as_f(bias, b_dt, v0 + c);
            store_from_f(dst, dst_dt, out_row + v0 + c, v);
            if (v_cache) v_pool[cache_base + (size_t)(c / hd) * head_stride + (c % hd)] = from_f<T>(v);
        }
    }
}

// The same with 16-byte accesses: a lane holds eight consecutive columns of a head (heads of up to 256 columns, a
// multiple of 8).  The pair of an interleaved rotation lies inside a lane; the partner of a half-split pair lies
// rot/16 lanes away and comes by shuffle.  Element types are read at run time (rows and pools of bfloat16 or float32).
__global__ void head_prep_vec_kernel(const void* src, int s_dt, long long lds, void* dst, int d_dt, long long ldd, int nq,
                                     int nk, int nv, int hd, int norm_dim, int rot, int interleaved,
                                     const void* __restrict__ bias, int b_dt, const void* __restrict__ wq,
                                     const void* __restrict__ wk, int w_dt, float eps, const float* __restrict__ inv_freq,
                                     const int* __restrict__ tok_pos, const int* __restrict__ tok_slot, void* k_pool,
                                     void* v_pool, const int* __restrict__ page_table, int max_pages, int page_size,
                                     int ring, const int* __restrict__ slot_len, int write_cache, int flags) {
    const int norm_whole = flags & QNN_PREP_WHOLE;
    const bool norm_last = flags & QNN_PREP_NORM_LAST, plain = flags & QNN_PREP_PLAIN_NORM;
    const bool v_is_k = flags & QNN_PREP_VALUES_ARE_KEYS;
    extern __shared__ float sm[];                   // [rot/2] (cos, sin) pairs, then [nq + nk] sums
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos != nullptr ? tok_pos[t] : 0;
    const int slot = tok_slot != nullptr ? tok_slot[t] : -1;
    const int rh = rot / 2;
    float2* angles = reinterpret_cast<float2*>(sm);
    for (int j = threadIdx.x; j < rh; j += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        angles[j] = make_float2(cs, sn);
    }
    __syncthreads();
    size_t cache_base = 0;
    bool wr = write_cache && slot >= 0;
    if (wr && ring > 0 && pos + ring < slot_len[slot]) wr = false;
    if (wr) {
        const int r = ring > 0 ? pos % ring : pos;
        const int page = page_table[(size_t)slot * max_pages + r / page_size];
        cache_base = ((size_t)page * nk * page_size + (r % page_size)) * hd;
    }
    const size_t head_stride = (size_t)page_size * hd;
    const size_t in_row = (size_t)t * lds, out_row = (size_t)t * ldd;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int col = lane * 8, shift = rh / 8;
    const bool active = col < hd;
    float inv_q = 0.f, inv_k = 0.f;
    if (norm_whole) {
        float* sums = sm + 2 * rh;
        for (int h = warp; h < nq + nk; h += nwarp) {
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (active) {
                load8_as_f(src, s_dt, in_row + (size_t)h * hd + col, v);
                if (bias != nullptr) {
                    float b[8];
                    load8_as_f(bias, b_dt, (size_t)h * hd + col, b);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] += b[e];
                }
            }
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (col + e < norm_dim) ss += v[e] * v[e];
            ss = warp_sum(ss);
            if (lane == 0) sums[h] = ss;
        }
        __syncthreads();
        float sq = 0.f, sk = 0.f;
        for (int h = 0; h < nq; ++h) sq += sums[h];
        for (int h = nq; h < nq + nk; ++h) sk += sums[h];
        inv_q = rsqrtf(sq / (float)(nq > 0 ? nq * norm_dim : 1) + eps);
        inv_k = rsqrtf(sk / (float)(nk > 0 ? nk * norm_dim : 1) + eps);
    }
    for (int h = warp; h < nq + nk; h += nwarp) {
        const bool is_k = h >= nq;
        const size_t c0 = (size_t)h * hd;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (active) {
            load8_as_f(src, s_dt, in_row + c0 + col, v);
            if (bias != nullptr) {
                float b[8];
                load8_as_f(bias, b_dt, c0 + col, b);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += b[e];
            }
        }
        const void* w = is_k ? wk : wq;
        const bool normed = w != nullptr || (plain && norm_dim > 0);
        if (is_k && v_is_k && active) {
            store8_from_f(dst, d_dt, out_row + (size_t)(h + nk) * hd + col, v);
            if (wr && v_pool != nullptr)
                store8_from_f(v_pool, d_dt, cache_base + (size_t)(h - nq) * head_stride + col, v);
        }
        auto norm = [&]() {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (col + e < norm_dim) ss += v[e] * v[e];
            ss = warp_sum(ss);
            const float inv = norm_whole ? (is_k ? inv_k : inv_q) : rsqrtf(ss / (float)norm_dim + eps);
            const size_t w0 = norm_whole ? (size_t)(is_k ? h - nq : h) * norm_dim : 0;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (col + e < norm_dim) v[e] = v[e] * inv * (w != nullptr ? load_as_f(w, w_dt, w0 + col + e) : 1.f);
        };
        if (normed && !norm_last) norm();
        if (rot > 0) {
            if (interleaved) {
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    if (col + e < rot) {
                        const float2 cs = angles[(col + e) >> 1];
                        const float a = v[e], b = v[e + 1];
                        v[e] = a * cs.x - b * cs.y;
                        v[e + 1] = b * cs.x + a * cs.y;
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float above = __shfl_down_sync(0xffffffffu, v[e], shift);     // column c + rot/2
                    const float below = __shfl_up_sync(0xffffffffu, v[e], shift);       // column c - rot/2
                    const int c = col + e;
                    if (c < rh) {
                        const float2 cs = angles[c];
                        v[e] = v[e] * cs.x - above * cs.y;
                    } else if (c < rot) {
                        const float2 cs = angles[c - rh];
                        v[e] = v[e] * cs.x + below * cs.y;
                    }
                }
            }
        }
        if (normed && norm_last) norm();
        if (active) {
            store8_from_f(dst, d_dt, out_row + c0 + col, v);
            if (is_k && wr) store8_from_f(k_pool, d_dt, cache_base + (size_t)(h - nq) * head_stride + col, v);
        }
    }
    const size_t v0 = (size_t)(nq + nk) * hd;
    const bool v_cache = wr && v_pool != nullptr;
    if (nv > 0 && !v_is_k && (bias != nullptr || v_cache || src != (const void*)dst)) {
        for (int c = threadIdx.x * 8; c < nv; c += blockDim.x * 8) {
            float v[8];
            load8_as_f(src, s_dt, in_row + v0 + c, v);
            if (bias != nullptr) {
                float b[8];
                load8_as_f(bias, b_dt, v0 + c, b);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += b[e];
            }
            store8_from_f(dst, d_dt, out_row + v0 + c, v);
            if (v_cache) store8_from_f(v_pool, d_dt, cache_base + (size_t)(c / hd) * head_stride + (c % hd), v);
        }
    }
}

}  // namespace

// src: [T, lds] rows of `dtype` holding nq query heads, nk key heads (hd columns each) and nv value columns, in that
// order; dst: the same layout with row pitch ldd in `dst_dt` (may be src itself).  bias: over the packed row, or null.
// wq / wk: norm weights [norm_dim] of `w_dt` (with norm_whole: [nq * norm_dim] and [nk * norm_dim]), or null.  inv_freq: [rot/2] float32.  The cache arguments are those of
// qnn_rope_cache_write; with write_cache, nv must be nk * hd (or 0 with v_pool null) and dst_dt the pools' type.
// flags: QNN_PREP_* (see the head of this file).
QNN_API int qnn_head_prep(const void* src, int dtype, long long lds, void* dst, int dst_dt, long long ldd, int T, int nq,
                          int nk, int nv, int hd, int norm_dim, int rot, int interleaved, const void* bias, int b_dt,
                          const void* wq, const void* wk, int w_dt, float eps, const float* inv_freq, const int* tok_pos,
                          const int* tok_slot, void* k_pool, void* v_pool, const int* page_table, int max_pages,
                          int page_size, int ring, const int* slot_len, int write_cache, int flags,
                          cudaStream_t st) {
    if (T <= 0) return 0;
    const int norm_whole = flags & QNN_PREP_WHOLE;
    if (nq < 0 || nk < 0 || nv < 0 || hd <= 0 || rot % 2 || rot < 0 || rot > hd || norm_dim < 0 || norm_dim > hd)
        return QNN_ERR_ARGUMENT;
    if ((wq != nullptr || wk != nullptr) && norm_dim == 0) return QNN_ERR_ARGUMENT;
    if (norm_whole && ((nq > 0 && wq == nullptr) || (nk > 0 && wk == nullptr))) return QNN_ERR_ARGUMENT;
    // a norm over all heads is formed before anything else: it cannot come after the rotation, nor go without weights
    if (norm_whole && (flags & (QNN_PREP_NORM_LAST | QNN_PREP_PLAIN_NORM))) return QNN_ERR_ARGUMENT;
    if ((flags & QNN_PREP_PLAIN_NORM) && (wq != nullptr || wk != nullptr)) return QNN_ERR_ARGUMENT;
    // values that are the keys: as many value columns as key columns, in a destination that is not the source
    if ((flags & QNN_PREP_VALUES_ARE_KEYS) && (nv != nk * hd || src == (const void*)dst)) return QNN_ERR_ARGUMENT;
    if (rot > 0 && (inv_freq == nullptr || tok_pos == nullptr)) return QNN_ERR_ARGUMENT;
    if (write_cache && (tok_slot == nullptr || k_pool == nullptr || page_table == nullptr || slot_len == nullptr ||
                        (v_pool != nullptr && nv != nk * hd)))
        return QNN_ERR_ARGUMENT;
    const int heads = nq + nk;
    int warps = heads >= 8 ? 8 : (heads >= 4 ? 4 : 2);
    if (T > 1024 && warps > 4) warps = 4;
    // 16-byte accesses where every piece starts on 16 bytes: heads, value columns and row pitches in whole pieces of 8
    // columns, heads of up to 256, a half-split rotation over a multiple of 16 columns
    const size_t es = dtype == QNN_DT_BF16 ? 2 : 4, ed = dst_dt == QNN_DT_BF16 ? 2 : 4;
    const bool aligned = ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0) && (lds * es) % 16 == 0 &&
                         (ldd * ed) % 16 == 0 && ((uintptr_t)bias % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) &&
                         ((uintptr_t)v_pool % 16 == 0);
    if (aligned && hd % 8 == 0 && hd <= 256 && nv % 8 == 0 && (interleaved ? rot % 2 == 0 : rot % 16 == 0)) {
        launch_pdl(head_prep_vec_kernel, dim3(T), dim3(warps * 32), ((size_t)rot + heads) * sizeof(float), st, src, dtype, lds,
                   dst, dst_dt, ldd, nq, nk, nv, hd, norm_dim, rot, interleaved, bias, b_dt, wq, wk, w_dt, eps, inv_freq,
                   tok_pos, tok_slot, k_pool, v_pool, page_table, max_pages, page_size, ring, slot_len, write_cache,
                   flags);
        QNN_LAUNCH_CHECK();
    }
    const size_t smem = ((size_t)rot + (size_t)warps * hd + heads) * sizeof(float);
    if (smem > 48 * 1024) return QNN_ERR_UNSUPPORTED;
    if (dtype == QNN_DT_BF16)
        launch_pdl(head_prep_kernel<bf16>, dim3(T), dim3(warps * 32), smem, st, (const bf16*)src, lds, dst, dst_dt, ldd, nq, nk,
                   nv, hd, norm_dim, rot, interleaved, bias, b_dt, wq, wk, w_dt, eps, inv_freq, tok_pos, tok_slot,
                   (bf16*)k_pool, (bf16*)v_pool, page_table, max_pages, page_size, ring, slot_len, write_cache, flags);
    else
        launch_pdl(head_prep_kernel<float>, dim3(T), dim3(warps * 32), smem, st, (const float*)src, lds, dst, dst_dt, ldd, nq,
                   nk, nv, hd, norm_dim, rot, interleaved, bias, b_dt, wq, wk, w_dt, eps, inv_freq, tok_pos, tok_slot,
                   (float*)k_pool, (float*)v_pool, page_table, max_pages, page_size, ring, slot_len, write_cache, flags);
    QNN_LAUNCH_CHECK();
}
