// Dynamic tanh, a norm that forms no mean and no variance:
//
//   y = tanh(alpha * x) * w + b            alpha: one learned number; w, b: one per column
//
//   qnn_dyt        y of every row, from float32 or bfloat16 rows, into either
//   qnn_add_dyt    resid += a (+ c), and then y = dyt(resid) in the same pass (w null: the add alone).  `a` is a
//                  sublayer's output in the activations' element type, `c` float32 rows (the embedded rows that a
//                  looped stack adds back before a pass); either may be null.
//   qnn_embed_dyt  the embedded rows (table[token] * scale, float32) and dyt of them in one pass
//
// Everything is elementwise and float32 between load and store (tanhf, not the approximation), so a row's numbers do
// not depend on the batch.  Four columns per thread with 16-byte accesses of the float32 stream where rows allow.
#include "common.cuh"

using namespace qnn;

namespace {

__device__ __forceinline__ float dyt(float x, float alpha, float w, float b) { return tanhf(alpha * x) * w + b; }

template <int V>
__global__ void add_dyt_kernel(float* __restrict__ resid, const void* __restrict__ a, int a_dt, const float* __restrict__ c,
                               float alpha, const void* __restrict__ w, int w_dt, const void* __restrict__ b, int b_dt,
                               void* __restrict__ out, int out_dt, int H, size_t n_vec) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const size_t e0 = i * V;
    const int col = (int)(e0 % (size_t)H);
    float x[V];
    if (V == 4) {
        const float4 r = *reinterpret_cast<const float4*>(resid + e0);
        x[0] = r.x; x[1] = r.y; x[2] = r.z; x[3] = r.w;
    } else {
        x[0] = resid[e0];
    }
    if (a != nullptr) {
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] += load_as_f(a, a_dt, e0 + j);
    }
    if (c != nullptr) {
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] += c[e0 + j];
    }
    if (a != nullptr || c != nullptr) {
        if (V == 4) *reinterpret_cast<float4*>(resid + e0) = make_float4(x[0], x[1], x[2], x[3]);
        else resid[e0] = x[0];
    }
    if (w == nullptr) return;
#pragma unroll
    for (int j = 0; j < V; ++j)
        store_from_f(out, out_dt, e0 + j, dyt(x[j], alpha, load_as_f(w, w_dt, col + j), load_as_f(b, b_dt, col + j)));
}

__global__ void dyt_kernel(const void* __restrict__ x, int x_dt, float alpha, const void* __restrict__ w, int w_dt,
                           const void* __restrict__ b, int b_dt, void* __restrict__ out, int out_dt, int H, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int col = (int)(i % (size_t)H);
    store_from_f(out, out_dt, i, dyt(load_as_f(x, x_dt, i), alpha, load_as_f(w, w_dt, col), load_as_f(b, b_dt, col)));
}

__global__ void embed_dyt_kernel(const int* __restrict__ tokens, const void* __restrict__ table, int t_dt, float scale,
                                 float alpha, const void* __restrict__ w, int w_dt, const void* __restrict__ b, int b_dt,
                                 float* __restrict__ x, void* __restrict__ out, int out_dt, int H, int vocab, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / (size_t)H;
    const int col = (int)(i - t * (size_t)H);
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const float v = load_as_f(table, t_dt, (size_t)tok * H + col) * scale;
    x[i] = v;
    if (w != nullptr) store_from_f(out, out_dt, i, dyt(v, alpha, load_as_f(w, w_dt, col), load_as_f(b, b_dt, col)));
}

}  // namespace

QNN_API int qnn_dyt(const void* x, int x_dt, float alpha, const void* w, int w_dt, const void* b, int b_dt, void* out,
                    int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0 || w == nullptr || b == nullptr) return QNN_ERR_ARGUMENT;
    const size_t n = (size_t)T * H;
    launch_pdl(dyt_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, x_dt, alpha, w, w_dt, b, b_dt, out, out_dt,
               H, n);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_add_dyt(float* resid, const void* a, int a_dt, const float* c, float alpha, const void* w, int w_dt,
                        const void* b, int b_dt, void* out, int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0 || (w != nullptr && (b == nullptr || out == nullptr))) return QNN_ERR_ARGUMENT;
    const size_t n = (size_t)T * H;
    if (H % 4 == 0 && ((uintptr_t)resid % 16) == 0) {
        launch_pdl(add_dyt_kernel<4>, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, st, resid, a, a_dt, c, alpha, w,
                   w_dt, b, b_dt, out, out_dt, H, n / 4);
    } else {
        launch_pdl(add_dyt_kernel<1>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, resid, a, a_dt, c, alpha, w, w_dt,
                   b, b_dt, out, out_dt, H, n);
    }
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_embed_dyt(const int* tokens, const void* table, int t_dt, float scale, float alpha, const void* w,
                          int w_dt, const void* b, int b_dt, float* x, void* out, int out_dt, int T, int H, int vocab,
                          cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0 || vocab <= 0 || (w != nullptr && (b == nullptr || out == nullptr))) return QNN_ERR_ARGUMENT;
    const size_t n = (size_t)T * H;
    launch_pdl(embed_dyt_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, tokens, table, t_dt, scale, alpha, w,
               w_dt, b, b_dt, x, out, out_dt, H, vocab, n);
    QNN_LAUNCH_CHECK();
}
