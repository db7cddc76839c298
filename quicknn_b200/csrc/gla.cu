// Gated linear attention: a matrix state per (sequence, head) that decays per key channel.
//
//   S_t = diag(a_t) S_{t-1} + k_t v_t^T          S: [dim, vdim], float32, kept per cache slot
//   o_t = S_t^T (q_t * q_scale)
//   a_t = sigmoid(z_t + bias)^(1/tau) = exp(log_sigmoid(z_t + bias) / tau)       (float32; formed by the kernel
//                                                  that forms z, see qnn_small_linear_f32)
//
//   qnn_gla_scan        walks the rows of every sequence of a step in order, from the slot's state and back
//                       into it: whole prompts, portions and single tokens are the same launch
//   qnn_gla_norm_gate   per head: RMS norm of o over vdim with a weight shared by the heads, times silu(g)
//
// The same scan serves matrix memories whose decay is one number per head (a constant, or a gate): `decay_per_head`
// reads decay[row, h] instead of decay[row, h*dim + i] (a row pitch of 0 gives every row the same decays), `kw`
// multiplies the key of (row, head) by a float32 weight (an input gate) as it is staged, and `ones_col` names a value
// column that is 1 in every row, so that its state column is the normaliser n_t = d_t n_{t-1} + w_t k_t and its output
// n_t . q_t.  `state_stride` is the distance between two slots' states in floats (a slot may keep more than S).
//
//   qnn_mlstm_gates     from the pre-activations of an input and a forget gate per (row, head): the soft-capped log
//                       gates, the running maximum m_t = max(f_t + m_{t-1}, i_t) from the slot's m and back into it,
//                       and per row the decay exp(f_t + m_{t-1} - m_t), the key weight exp(i_t - m_t) and exp(-m_t)
//   qnn_head_norm_gate  qnn_gla_norm_gate with its options: a denominator max(|n.q|, e) + 1e-6 first, the norm's weight
//                       per column of a head, per column of the row, or none, and silu or sigmoid of the gate
//
// The scan: a block owns 64 (32 with more than 128 key channels) value columns of one (sequence, head).  Eight lanes
// share a group of 4 (2) columns, each with an eighth of the key channels of the state in registers, so that what a
// lane reads of q, k and the decay from shared memory serves several columns (with one column per lane the kernel
// was bound by shared-memory bandwidth: every column read the same 1.5 KB per row).  q, k, the decay and v of 16 rows
// at a time are staged in shared memory, the next 16 rows' loads in flight while these are walked.  The order of
// the sums depends on dim only, so a row gives the same numbers in any batch and any cutting of its sequence.
#include "common.cuh"

using namespace qnn;

namespace {

constexpr int GLA_SHARE = 8;      // lanes that share a group of columns, each with an eighth of the key channels
constexpr int GLA_ROWS = 16;      // rows staged at a time
constexpr int GLA_THREADS = 128;
constexpr int GLA_GROUPS = GLA_THREADS / GLA_SHARE;      // column groups of a block

// One chunk of GLA_ROWS rows in shared memory: q, k, decay as [row][part][channel of the part] with a pad of 4 floats
// between the parts (the eight lanes of a column group read 16 bytes each from eight different banks), then v
// [row][column].  RPT: key channels per lane; CPT: value columns per lane.
template <int RPT, int CPT>
struct GlaChunk {
    static constexpr int COLS = GLA_GROUPS * CPT;
    static constexpr int PART = RPT + 4, ROW = GLA_SHARE * PART, ARRAY = GLA_ROWS * ROW;
    static constexpr int FLOATS = 3 * ARRAY + GLA_ROWS * COLS;
    static constexpr int PER_THREAD = GLA_ROWS * RPT * GLA_SHARE / GLA_THREADS;      // staged elements of one array per thread
    static constexpr int V_PER_THREAD = GLA_ROWS * COLS / GLA_THREADS;
};

template <typename T, int RPT, int CPT>
__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                const float* __restrict__ decay, long long ldd, float q_scale, const int* __restrict__ seq_row0,
                const int* __restrict__ seq_len, const int* __restrict__ slots, float* __restrict__ state,
                float* __restrict__ out, long long ldo, int H, int dim, int vdim, int seg_len, int nseg,
                int decay_per_head, const float* __restrict__ kw, long long ldw, int ones_col, long long state_stride,
                int key_from_decay) {
    using C = GlaChunk<RPT, CPT>;
    constexpr int DIMP = RPT * GLA_SHARE;                    // key channels with padding
    constexpr bool AHEAD = RPT <= 16;                        // the next chunk's loads in registers while this one is walked
    extern __shared__ __align__(16) float sm[];
    const int h = blockIdx.y, c0 = blockIdx.x * C::COLS;
    pdl_wait();
    // whole sequences: block z walks sequence z from its slot's state.  Segments (seg_len > 0): block z walks segment
    // z % nseg of sequence z / nseg, rows seg * seg_len .. of it, from and into entry z of `state` (a scratch)
    int slot, row0, n;
    if (seg_len > 0) {
        const int b = blockIdx.z / nseg, seg = blockIdx.z - b * nseg;
        const int len = seq_len ? seq_len[b] : 1;
        slot = slots[b] >= 0 ? (int)blockIdx.z : -1;
        row0 = (seq_row0 ? seq_row0[b] : b) + seg * seg_len;
        n = max(0, min(seg_len, len - seg * seg_len));
    } else {
        slot = slots[blockIdx.z];
        row0 = seq_row0 ? seq_row0[blockIdx.z] : blockIdx.z;
        n = seq_len ? seq_len[blockIdx.z] : 1;
    }
    const int part = threadIdx.x & (GLA_SHARE - 1), grp = threadIdx.x / GLA_SHARE;
    const int col = c0 + grp * CPT;                          // the first of this lane's columns
    float S[RPT][CPT];
    float* my_state = state + (size_t)(slot < 0 ? 0 : slot) * state_stride + ((size_t)h * dim) * vdim + col;
    const int vreal = vdim - (ones_col >= 0 ? 1 : 0);       // value columns that the rows really hold
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int i = part * RPT + r;
            S[r][c] = (slot >= 0 && i < dim && col + c < vdim) ? my_state[(size_t)i * vdim + c] : 0.f;
        }
    // what is loaded stays as it came until `put`: a conversion here would wait for the load at once, and the loads
    // are meant to be in flight while the rows before them are walked
    T rq[C::PER_THREAD], rk[C::PER_THREAD], rv[C::V_PER_THREAD];
    float ra[C::PER_THREAD], rw[C::PER_THREAD];
    auto fetch = [&](int t0) {                               // global memory -> registers (rows beyond the sequence: nothing)
        const int nt = min(GLA_ROWS, n - t0);
#pragma unroll
        for (int e = 0; e < C::PER_THREAD; ++e) {
            const int idx = threadIdx.x + e * GLA_THREADS, tt = idx / DIMP, i = idx - tt * DIMP;
            rq[e] = from_f<T>(0.f); rk[e] = from_f<T>(0.f); ra[e] = 1.f; rw[e] = 1.f;
            if (tt < nt && i < dim) {
                const size_t row = (size_t)(row0 + t0 + tt);
                rq[e] = q[row * ld + h * dim + i];
                if (!key_from_decay) rk[e] = k[row * ld + h * dim + i];
                ra[e] = decay[row * ldd + (decay_per_head ? h : h * dim + i)];
                if (kw != nullptr) rw[e] = kw[row * ldw + h];
            }
        }
#pragma unroll
        for (int e = 0; e < C::V_PER_THREAD; ++e) {
            const int idx = threadIdx.x + e * GLA_THREADS, tt = idx / C::COLS, c = idx - tt * C::COLS;
            rv[e] = from_f<T>(0.f);
            if (tt < nt && c0 + c < vdim)
                rv[e] = c0 + c == ones_col ? from_f<T>(1.f) : v[(size_t)(row0 + t0 + tt) * ld + h * vreal + c0 + c];
        }
    };
    auto put = [&](float* buf) {                             // registers -> shared memory
#pragma unroll
        for (int e = 0; e < C::PER_THREAD; ++e) {
            const int idx = threadIdx.x + e * GLA_THREADS, tt = idx / DIMP, i = idx - tt * DIMP;
            const int at = tt * C::ROW + (i / RPT) * C::PART + (i % RPT);
            buf[at] = to_f(rq[e]) * q_scale;
            // key_from_decay: the key is what the decay leaves room for, 1 - a, in float32 (rows and channels beyond the
            // sequence's have a = 1 and so a key of 0)
            buf[C::ARRAY + at] = (key_from_decay ? 1.f - ra[e] : to_f(rk[e])) * rw[e];
            buf[2 * C::ARRAY + at] = ra[e];
        }
#pragma unroll
        for (int e = 0; e < C::V_PER_THREAD; ++e) buf[3 * C::ARRAY + threadIdx.x + e * GLA_THREADS] = to_f(rv[e]);
    };
    fetch(0);
    put(sm);
    __syncthreads();
    int cur = 0;
    for (int t0 = 0; t0 < n; t0 += GLA_ROWS) {
        const int nt = min(GLA_ROWS, n - t0);
        const bool more = t0 + GLA_ROWS < n;
        float* buf = sm + (AHEAD ? cur * C::FLOATS : 0);
        if (AHEAD && more) fetch(t0 + GLA_ROWS);
        for (int tt = 0; tt < nt; ++tt) {
            float vj[CPT], acc[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                vj[c] = buf[3 * C::ARRAY + tt * C::COLS + grp * CPT + c];
                acc[c] = 0.f;
            }
            const float4* aq = reinterpret_cast<const float4*>(buf + tt * C::ROW + part * C::PART);
            const float4* ak = reinterpret_cast<const float4*>(buf + C::ARRAY + tt * C::ROW + part * C::PART);
            const float4* aa = reinterpret_cast<const float4*>(buf + 2 * C::ARRAY + tt * C::ROW + part * C::PART);
#pragma unroll
            for (int j = 0; j < RPT / 4; ++j) {
                const float4 a4 = aa[j], k4 = ak[j], q4 = aq[j];
                const float av[4] = {a4.x, a4.y, a4.z, a4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w};
                const float qv[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        S[4 * j + u][c] = av[u] * S[4 * j + u][c] + kv[u] * vj[c];
                        acc[c] += S[4 * j + u][c] * qv[u];
                    }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 4);
                if (out != nullptr && part == 0 && col + c < vdim)
                    out[(size_t)(row0 + t0 + tt) * ldo + h * vdim + col + c] = slot >= 0 ? acc[c] : 0.f;
            }
        }
        if (more) {
            if (AHEAD) {
                put(sm + (cur ^ 1) * C::FLOATS);             // nobody reads that buffer: its chunk was walked a round ago
                cur ^= 1;
            } else {
                __syncthreads();
                fetch(t0 + GLA_ROWS);
                put(sm);
            }
            __syncthreads();
        }
    }
    if (slot >= 0) {
#pragma unroll
        for (int r = 0; r < RPT; ++r)
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int i = part * RPT + r;
                if (i < dim && col + c < vdim) my_state[(size_t)i * vdim + c] = S[r][c];
            }
    }
}

// ---- long prompts in segments ------------------------------------------------------------------------------------
// The recurrence is linear in the state: over a segment of rows, S_end = D (.) S_start + L with D the product of the
// segment's decays per key channel and L the state that the segment builds from nothing.  So a long sequence is cut
// into segments of seg_len rows that run side by side: the scan once without outputs from empty states (L), the
// decay products (D), a short pass over the segments in order that leaves every segment's start state in the scratch
// and the sequence's new state in its slot, and the scan once more from those start states, with outputs.

// D[z][c] = product of decay[rows of segment z][c]; a thread per (segment, channel)
__global__ void gla_segment_decay_kernel(const float* __restrict__ decay, long long ldd, const int* __restrict__ seq_row0,
                                         const int* __restrict__ seq_len, int seg_len, int nseg, float* __restrict__ D,
                                         int HD) {
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, z = blockIdx.y;
    if (c >= HD) return;
    const int b = z / nseg, seg = z - b * nseg;
    const int row0 = seq_row0[b] + seg * seg_len, n = max(0, min(seg_len, seq_len[b] - seg * seg_len));
    float d = 1.f;
    for (int t = 0; t < n; ++t) d *= decay[(size_t)(row0 + t) * ldd + c];
    D[(size_t)z * HD + c] = d;
}

// scratch[z] holds L of segment z and gets the segment's start state; the slot's state moves on to the sequence's end.
// A thread per state element of a sequence.
__global__ void gla_segment_prefix_kernel(float* __restrict__ scratch, const float* __restrict__ D,
                                          const int* __restrict__ slots, float* __restrict__ state, int nseg, int dim,
                                          int vdim, size_t per_seq, int decay_per_head, long long state_stride) {
    pdl_wait();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (e >= per_seq) return;
    const int slot = slots[b];
    if (slot < 0) return;
    // the decay's column: (head, key channel), or the head alone
    const size_t hi = decay_per_head ? e / ((size_t)dim * vdim) : e / vdim;
    const size_t n_dec = decay_per_head ? per_seq / ((size_t)dim * vdim) : per_seq / vdim;
    float carry = state[(size_t)slot * state_stride + e];
    for (int seg = 0; seg < nseg; ++seg) {
        const size_t z = (size_t)b * nseg + seg;
        const float L = scratch[z * per_seq + e];
        scratch[z * per_seq + e] = carry;
        carry = D[z * n_dec + hi] * carry + L;
    }
    state[(size_t)slot * state_stride + e] = carry;
}

// a warp per (row, head).  o: float32 rows of H heads, `hs` columns apart, of which the first vdim are normed; with `den`
// (float32 [rows, ldden], one per head) a head is first divided by max(|o[vdim]|, den) + 1e-6, o[vdim] being the
// normaliser's product with the query.  w_mode: 0 no weight, 1 a weight per column of a head (shared by the heads),
// 2 a weight per column of the row.  gate_act: 0 silu, 1 sigmoid.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, long long ldo, int hs, const float* __restrict__ den,
                                      long long ldden, const void* __restrict__ w, int w_dt, int w_mode, float eps,
                                      const T* __restrict__ g, long long ldg, int gate_act, T* __restrict__ out,
                                      long long ld_out, int rows, int H, int vdim) {
    pdl_wait();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= rows * H) return;
    const int t = unit / H, h = unit - t * H;
    const float* orow = o + (size_t)t * ldo + (size_t)h * hs;
    float scale = 1.f;
    if (den != nullptr) scale = 1.f / (fmaxf(fabsf(orow[vdim]), den[(size_t)t * ldden + h]) + 1e-6f);
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) {
        const float v = orow[j] * scale;
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
        const float gv = gate_act == 2 ? 0.f : to_f(g[(size_t)t * ldg + h * vdim + j]);
        const float wv = w_mode == 0 ? 1.f : load_as_f(w, w_dt, w_mode == 2 ? (size_t)h * vdim + j : (size_t)j);
        const float ga = gate_act == 2 ? 1.f : (gate_act == 1 ? 1.f / (1.f + expf(-gv)) : silu(gv));
        out[(size_t)t * ld_out + h * vdim + j] = from_f<T>(orow[j] * scale * inv * wv * ga);
    }
}

// The same for heads so wide that a warp would walk them for long (one norm over all heads of a row, handed in as a
// single head): a block per (row, head), the row's sum by all its warps in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_wide_kernel(const float* __restrict__ o, long long ldo, int hs, const float* __restrict__ den,
                           long long ldden, const void* __restrict__ w, int w_dt, int w_mode, float eps,
                           const T* __restrict__ g, long long ldg, int gate_act, T* __restrict__ out, long long ld_out,
                           int rows, int H, int vdim) {
    __shared__ float red[32];
    pdl_wait();
    const int unit = blockIdx.x;
    const int t = unit / H, h = unit - t * H;
    const float* orow = o + (size_t)t * ldo + (size_t)h * hs;
    float scale = 1.f;
    if (den != nullptr) scale = 1.f / (fmaxf(fabsf(orow[vdim]), den[(size_t)t * ldden + h]) + 1e-6f);
    float ss = 0.f;
    for (int j = threadIdx.x; j < vdim; j += blockDim.x) {
        const float v = orow[j] * scale;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)vdim + eps);
    for (int j = threadIdx.x; j < vdim; j += blockDim.x) {
        const float gv = gate_act == 2 ? 0.f : to_f(g[(size_t)t * ldg + h * vdim + j]);
        const float wv = w_mode == 0 ? 1.f : load_as_f(w, w_dt, w_mode == 2 ? (size_t)h * vdim + j : (size_t)j);
        const float ga = gate_act == 2 ? 1.f : (gate_act == 1 ? 1.f / (1.f + expf(-gv)) : silu(gv));
        out[(size_t)t * ld_out + h * vdim + j] = from_f<T>(orow[j] * scale * inv * wv * ga);
    }
}

// ---- gates of a matrix memory with a running maximum ---------------------------------------------------------------
// pre: float32 [rows, ldp] with the input gate's pre-activation of head h at column h and the forget gate's at H + h;
// bias: [2H] (input gates, then forget gates).  i = cap tanh((pre_i + b_i) / cap); f = log sigmoid(cap tanh((pre_f +
// b_f) / cap)).  A warp takes 32 rows at a time: every lane forms one row's log gates (the hyperbolic tangents, the
// logarithm), then all lanes walk m_t = max(f_t + m_{t-1}, i_t) through the 32 rows in order.  gates: float32 [rows, 3H]: the decay exp(f_t + m_{t-1} - m_t), the key weight exp(i_t - m_t),
// exp(-m_t).  A warp per (sequence, head); m of the slot's head at mstate[slot * state_stride + h].
__global__ void mlstm_gates_kernel(const float* __restrict__ pre, long long ldp, const void* __restrict__ bias, int b_dt,
                                   float cap, const int* __restrict__ seq_row0, const int* __restrict__ seq_len,
                                   const int* __restrict__ slots, float* __restrict__ mstate, long long state_stride,
                                   float* __restrict__ gates, int H, int B) {
    pdl_wait();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= B * H) return;
    const int b = unit / H, h = unit - b * H;
    const int slot = slots[b];
    const int row0 = seq_row0 ? seq_row0[b] : b, n = seq_len ? seq_len[b] : 1;
    const float bi = load_as_f(bias, b_dt, h), bf = load_as_f(bias, b_dt, H + h);
    float m = slot >= 0 ? mstate[(size_t)slot * state_stride + h] : 0.f;
    const size_t ldg = (size_t)3 * H;
    for (int t0 = 0; t0 < n; t0 += 32) {
        const int t = t0 + lane;
        float gi = -INFINITY, gf = 0.f;                        // rows beyond the sequence change nothing: m -> max(m, -inf)
        if (t < n) {
            const float zi = pre[(size_t)(row0 + t) * ldp + h] + bi, zf = pre[(size_t)(row0 + t) * ldp + H + h] + bf;
            gi = cap * tanhf(zi / cap);
            const float c = cap * tanhf(zf / cap);
            gf = fminf(c, 0.f) - log1pf(expf(-fabsf(c)));
        }
        // the rows of the chunk in order; every lane walks them all, so m is the same bit for bit whether a row came
        // in a prompt, in a portion or alone
        float before = m, mt = m;
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
            const float fj = __shfl_sync(0xffffffffu, gf, j), ij = __shfl_sync(0xffffffffu, gi, j);
            const float next = fmaxf(m + fj, ij);
            if (lane == j) {
                before = m;
                mt = next;
            }
            m = next;
        }
        if (t < n) {
            float* gr = gates + (size_t)(row0 + t) * ldg;
            const bool live = slot >= 0;
            gr[h] = live ? expf(gf + before - mt) : 0.f;
            gr[H + h] = live ? expf(gi - mt) : 0.f;
            gr[2 * H + h] = live ? expf(-mt) : 1.f;
        }
    }
    if (slot >= 0 && lane == 0) mstate[(size_t)slot * state_stride + h] = m;
}

// Gates of a matrix memory whose forget gate also decides what is written.  rows: [T, ld] of T with the query columns
// (nq of them, from column q_col) and the forget gate's pre-activations (nf, from column f_col).  The queries get
// silu in place; f = l + (1 - l) sigmoid(z + bias), float32, goes to `f_out` [T, nf] (l: a lower bound per channel).
template <typename T>
__global__ void bounded_gates_kernel(T* __restrict__ rows, long long ld, int q_col, int nq, int f_col, int nf,
                                     const void* __restrict__ bias, int b_dt, const void* __restrict__ lower, int l_dt,
                                     float* __restrict__ f_out, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / (size_t)(nq + nf);
    const int c = (int)(i - t * (size_t)(nq + nf));
    if (c < nq) {
        T* at = rows + t * ld + q_col + c;
        *at = from_f<T>(silu(to_f(*at)));
    } else {
        const int j = c - nq;
        const float z = to_f(rows[t * ld + f_col + j]) + (bias != nullptr ? load_as_f(bias, b_dt, j) : 0.f);
        const float l = lower != nullptr ? load_as_f(lower, l_dt, j) : 0.f;
        f_out[t * nf + j] = l + (1.f - l) * (1.f / (1.f + expf(-z)));
    }
}

struct ScanExtra {
    int decay_per_head = 0;
    const float* kw = nullptr;
    long long ldw = 0;
    int ones_col = -1;
    long long state_stride = 0;         // 0: H * dim * vdim
    int key_from_decay = 0;             // the keys are 1 - decay (per key channel), k is not read
};

template <typename T>
int scan_launch(const void* q, const void* k, const void* v, long long ld, const float* decay, long long ldd, float q_scale,
                const int* seq_row0, const int* seq_len, const int* slots, float* state, float* out, long long ldo, int B,
                int H, int dim, int vdim, int seg_len, int nseg, cudaStream_t st, ScanExtra x = ScanExtra()) {
    const int rpt = (dim + GLA_SHARE - 1) / GLA_SHARE;
    const long long stride = x.state_stride > 0 ? x.state_stride : (long long)H * dim * vdim;
#define QNN_GLA(RPTV, CPTV)                                                                                          \
    {                                                                                                                \
        using C = GlaChunk<RPTV, CPTV>;                                                                              \
        const dim3 grid((vdim + C::COLS - 1) / C::COLS, H, seg_len > 0 ? B * nseg : B);                              \
        const size_t smem = (size_t)C::FLOATS * sizeof(float) * (RPTV <= 16 ? 2 : 1);                                \
        static bool set = false;                                                                                     \
        if (smem > 48 * 1024 && !set) {                                                                              \
            cudaFuncSetAttribute(gla_scan_kernel<T, RPTV, CPTV>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                 (int)smem);                                                                         \
            set = true;                                                                                              \
        }                                                                                                            \
        launch_pdl(gla_scan_kernel<T, RPTV, CPTV>, grid, dim3(GLA_THREADS), smem, st, (const T*)q, (const T*)k,     \
                   (const T*)v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, H, dim, vdim,    \
                   seg_len, nseg, x.decay_per_head, x.kw, x.ldw, x.ones_col, stride, x.key_from_decay);             \
    }
    if (rpt <= 4) QNN_GLA(4, 4)
    else if (rpt <= 8) QNN_GLA(8, 4)
    else if (rpt <= 16) QNN_GLA(16, 4)
    else if (rpt <= 32) QNN_GLA(32, 2)
    else return QNN_ERR_UNSUPPORTED;
#undef QNN_GLA
    QNN_LAUNCH_CHECK();
}

template <typename T>
int scan_segments(const void* q, const void* k, const void* v, long long ld, const float* decay, long long ldd, float q_scale,
                  const int* seq_row0, const int* seq_len, const int* slots, float* state, float* out, long long ldo, int B,
                  int H, int dim, int vdim, int seg_len, int nseg, float* scratch, float* seg_decay, cudaStream_t st,
                  ScanExtra x = ScanExtra()) {
    const size_t per_seq = (size_t)H * dim * vdim;
    const long long slot_stride = x.state_stride > 0 ? x.state_stride : (long long)per_seq;
    ScanExtra in_scratch = x;
    in_scratch.state_stride = (long long)per_seq;            // segment z's state is entry z of the scratch
    int rc = scan_launch<T>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, scratch, nullptr, ldo, B, H, dim, vdim,
                            seg_len, nseg, st, in_scratch);
    if (rc != 0) return rc;
    const int HD = x.decay_per_head ? H : H * dim;
    launch_pdl(gla_segment_decay_kernel, dim3((HD + 127) / 128, B * nseg), dim3(128), 0, st, decay, ldd, seq_row0, seq_len,
               seg_len, nseg, seg_decay, HD);
    launch_pdl(gla_segment_prefix_kernel, dim3((unsigned)((per_seq + 255) / 256), B), dim3(256), 0, st, scratch,
               (const float*)seg_decay, slots, state, nseg, dim, vdim, per_seq, x.decay_per_head, slot_stride);
    if ((rc = (int)cudaGetLastError()) != 0) return rc;
    return scan_launch<T>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, scratch, out, ldo, B, H, dim, vdim,
                          seg_len, nseg, st, in_scratch);
}

}  // namespace

// q, k: [rows, H*dim] and v: [rows, H*vdim] of `dtype`, one row pitch `ld` (pieces of one stacked product);
// decay: the decays a [rows, H*dim] float32 (qnn_small_linear_f32 forms them in its epilogue); seq_row0 / seq_len:
// first row and row count of each of the B sequences (both null: sequence b is row b alone); slots: the state slot
// of each sequence, negative for a row of no sequence (its output is zero, no state is touched); state:
// [slots, H, dim, vdim] float32; out: [rows, H*vdim] float32.  dim up to 256.
// key_from_decay != 0: the keys are 1 - decay, formed in float32 as the rows are staged; k is not read (may be null).
QNN_API int qnn_gla_scan(const void* q, const void* k, const void* v, long long ld, int dtype, const float* decay,
                         long long ldd, float q_scale, const int* seq_row0, const int* seq_len, const int* slots,
                         float* state, float* out, long long ldo, int B, int H, int dim, int vdim, int key_from_decay,
                         cudaStream_t st) {
    if (B <= 0) return 0;
    if (H <= 0 || dim <= 0 || vdim <= 0 || H > 65535 || B > 65535) return QNN_ERR_ARGUMENT;
    if ((seq_row0 == nullptr) != (seq_len == nullptr)) return QNN_ERR_ARGUMENT;
    ScanExtra x;
    x.key_from_decay = key_from_decay ? 1 : 0;
    if (dtype == QNN_DT_BF16)
        return scan_launch<bf16>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim,
                                 vdim, 0, 1, st, x);
    return scan_launch<float>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim, vdim,
                              0, 1, st, x);
}

// The same for sequences of up to nseg * seg_len rows, in segments that run side by side (see above).  scratch:
// [B * nseg, H, dim, vdim] float32, zeroed by the caller; seg_decay: [B * nseg, H * dim] float32.  Four launches.
QNN_API int qnn_gla_scan_segments(const void* q, const void* k, const void* v, long long ld, int dtype, const float* decay,
                                  long long ldd, float q_scale, const int* seq_row0, const int* seq_len, const int* slots,
                                  float* state, float* out, long long ldo, int B, int H, int dim, int vdim, int seg_len,
                                  int nseg, float* scratch, float* seg_decay, int key_from_decay, cudaStream_t st) {
    if (B <= 0) return 0;
    if (H <= 0 || dim <= 0 || vdim <= 0 || H > 65535 || seg_len < 1 || nseg < 1 || (long long)B * nseg > 65535)
        return QNN_ERR_ARGUMENT;
    if (seq_row0 == nullptr || seq_len == nullptr) return QNN_ERR_ARGUMENT;
    ScanExtra x;
    x.key_from_decay = key_from_decay ? 1 : 0;
    if (dtype == QNN_DT_BF16)
        return scan_segments<bf16>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim,
                                   vdim, seg_len, nseg, scratch, seg_decay, st, x);
    return scan_segments<float>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim, vdim,
                                seg_len, nseg, scratch, seg_decay, st, x);
}

// The scan with one decay per (row, head): S_t = d_t S_{t-1} + w_t k_t v_t^T, o_t = S_t^T (q_t q_scale).
// decay: float32, decay[row * ldd + h] (ldd = 0: the same H decays in every row); kw: the key weights w,
// kw[row * ldw + h], or null for 1.  normaliser != 0: the state has one column more than the rows have value columns,
// which is fed 1 in every row (n_t = d_t n_{t-1} + w_t k_t); out then has vdim + 1 columns per head, the last n_t . q_t.
// state: the slot's [H, dim, vdim (+1)] floats start at state + slot * state_stride.  seg_len > 0: in segments, with
// scratch [B * nseg, H, dim, vdim (+1)] zeroed by the caller and seg_decay [B * nseg, H].
QNN_API int qnn_memory_scan(const void* q, const void* k, const void* v, long long ld, int dtype, const float* decay,
                            long long ldd, const float* kw, long long ldw, float q_scale, int normaliser,
                            const int* seq_row0, const int* seq_len, const int* slots, float* state, long long state_stride,
                            float* out, long long ldo, int B, int H, int dim, int vdim, int seg_len, int nseg,
                            float* scratch, float* seg_decay, cudaStream_t st) {
    if (B <= 0) return 0;
    if (H <= 0 || dim <= 0 || vdim <= 0 || H > 65535 || B > 65535) return QNN_ERR_ARGUMENT;
    if ((seq_row0 == nullptr) != (seq_len == nullptr)) return QNN_ERR_ARGUMENT;
    const int vs = vdim + (normaliser ? 1 : 0);
    if (state_stride < (long long)H * dim * vs) return QNN_ERR_ARGUMENT;
    ScanExtra x;
    x.decay_per_head = 1;
    x.kw = kw;
    x.ldw = ldw;
    x.ones_col = normaliser ? vdim : -1;
    x.state_stride = state_stride;
    if (seg_len > 0) {
        if (nseg < 1 || (long long)B * nseg > 65535 || seq_row0 == nullptr || scratch == nullptr || seg_decay == nullptr)
            return QNN_ERR_ARGUMENT;
        if (dtype == QNN_DT_BF16)
            return scan_segments<bf16>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim,
                                       vs, seg_len, nseg, scratch, seg_decay, st, x);
        return scan_segments<float>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim,
                                    vs, seg_len, nseg, scratch, seg_decay, st, x);
    }
    if (dtype == QNN_DT_BF16)
        return scan_launch<bf16>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim, vs,
                                 0, 1, st, x);
    return scan_launch<float>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim, vs, 0,
                              1, st, x);
}

QNN_API int qnn_mlstm_gates(const float* pre, long long ldp, const void* bias, int b_dt, float cap, const int* seq_row0,
                            const int* seq_len, const int* slots, float* mstate, long long state_stride, float* gates,
                            int H, int B, cudaStream_t st) {
    if (B <= 0) return 0;
    if (H <= 0 || !(cap > 0.f) || (seq_row0 == nullptr) != (seq_len == nullptr)) return QNN_ERR_ARGUMENT;
    const int warps = 4;
    launch_pdl(mlstm_gates_kernel, dim3(((size_t)B * H + warps - 1) / warps), dim3(warps * 32), 0, st, pre, ldp, bias, b_dt,
               cap, seq_row0, seq_len, slots, mstate, state_stride, gates, H, B);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_head_norm_gate(const float* o, long long ldo, int hs, const float* den, long long ldden, const void* w,
                               int w_dt, int w_mode, float eps, const void* g, long long ldg, int gate_act, void* out,
                               long long ld_out, int dtype, int rows, int H, int vdim, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (H <= 0 || vdim <= 0 || hs < vdim || (den != nullptr && hs <= vdim) || (w_mode != 0 && w == nullptr))
        return QNN_ERR_ARGUMENT;
    if (gate_act < 0 || gate_act > 2 || (gate_act != 2 && g == nullptr)) return QNN_ERR_ARGUMENT;      // 2: no gate
    if (vdim >= 512 && (long long)rows * H <= 0x7fffffffLL) {         // a block per (row, head)
        const dim3 wide((unsigned)(rows * H));
        if (dtype == QNN_DT_BF16)
            launch_pdl(head_norm_gate_wide_kernel<bf16>, wide, dim3(256), 0, st, o, ldo, hs, den, ldden, w, w_dt, w_mode, eps,
                       (const bf16*)g, ldg, gate_act, (bf16*)out, ld_out, rows, H, vdim);
        else
            launch_pdl(head_norm_gate_wide_kernel<float>, wide, dim3(256), 0, st, o, ldo, hs, den, ldden, w, w_dt, w_mode, eps,
                       (const float*)g, ldg, gate_act, (float*)out, ld_out, rows, H, vdim);
        QNN_LAUNCH_CHECK();
    }
    const int warps = 4;
    const dim3 grid(((size_t)rows * H + warps - 1) / warps);
    if (dtype == QNN_DT_BF16)
        launch_pdl(head_norm_gate_kernel<bf16>, grid, dim3(warps * 32), 0, st, o, ldo, hs, den, ldden, w, w_dt, w_mode, eps,
                   (const bf16*)g, ldg, gate_act, (bf16*)out, ld_out, rows, H, vdim);
    else
        launch_pdl(head_norm_gate_kernel<float>, grid, dim3(warps * 32), 0, st, o, ldo, hs, den, ldden, w, w_dt, w_mode, eps,
                   (const float*)g, ldg, gate_act, (float*)out, ld_out, rows, H, vdim);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_bounded_gates(void* rows, int dtype, long long ld, int T, int q_col, int nq, int f_col, int nf,
                              const void* bias, int b_dt, const void* lower, int l_dt, float* f_out, cudaStream_t st) {
    if (T <= 0) return 0;
    if (nq < 0 || nf <= 0 || q_col < 0 || f_col < 0 || f_out == nullptr) return QNN_ERR_ARGUMENT;
    const size_t n = (size_t)T * (nq + nf);
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == QNN_DT_BF16)
        launch_pdl(bounded_gates_kernel<bf16>, grid, dim3(256), 0, st, (bf16*)rows, ld, q_col, nq, f_col, nf, bias, b_dt,
                   lower, l_dt, f_out, n);
    else
        launch_pdl(bounded_gates_kernel<float>, grid, dim3(256), 0, st, (float*)rows, ld, q_col, nq, f_col, nf, bias, b_dt,
                   lower, l_dt, f_out, n);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_gla_norm_gate(const float* o, long long ldo, const void* w, int w_dt, float eps, const void* g,
                              long long ldg, void* out, long long ld_out, int dtype, int rows, int H, int vdim,
                              cudaStream_t st) {
    return qnn_head_norm_gate(o, ldo, vdim, nullptr, 0, w, w_dt, 1, eps, g, ldg, 0, out, ld_out, dtype, rows, H, vdim, st);
}
