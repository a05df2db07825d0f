// Kernels around gated mixers and gated side inputs, for float and bfloat16 activations (A):
//   qk_norm_store    RMS norm of the whole query projection and of the whole key projection (all heads at once),
//                    rotation by position, queries out, keys and values into the paged cache
//   head_gate        attention output of every head times the sigmoid of that head's gate logit
//   add_cast         residual stream += pending addend; a copy of the stream in the element type
//   gelu_mul_rows    gelu(a) times a slice of a per-token table row
//   add_rms_normed   residual stream += y / rms(y) * w
//   softcap          cap * tanh(x / cap) in place
// Norms, sums of squares, angles, sigmoids and the residual sum are float whatever A is.
#pragma once
#include "common.cuh"

namespace gate {

template <typename A> __device__ __forceinline__ float ld_flag(const void* p, int is_f32, size_t i) {
  return is_f32 ? ((const float*)p)[i] : to_f32(((const A*)p)[i]);
}
__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_tanh_f(float v) {
  return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

// ------------------------------------------------------------------ query/key norm, rotation, cache write
// Row t of c (float or A, row stride ld) holds [H query heads of hd | G key heads of hd | G value heads of vd].
// With qw / kw (norm weights over H * hd and G * hd columns; either may be null) the query part and the key part
// are each divided by their root mean square over ALL their columns and multiplied by the weight. Then the
// first `rot` dims of every query and key head turn by the token's position (table cs[pos][i] = (cos, sin);
// half pairing i with i + rot / 2, or adjacent pairs), queries go to q_out [T, ldq], keys and values to the
// token's place in the cache pages. G == 0: queries only.
template <typename A>
__global__ void __launch_bounds__(256) qk_norm_store_kernel(const void* __restrict__ c, int c_f32, int ld, A* __restrict__ q_out,
                                                            int ldq, const int* __restrict__ tok_pos,
                                                            const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                                            int max_pages, const float2* __restrict__ cs, A* __restrict__ kpages,
                                                            A* __restrict__ vpages, int H, int G, int hd, int vd, int rot,
                                                            int interleaved, const void* __restrict__ qw,
                                                            const void* __restrict__ kw, int w_f32, float eps) {
  __shared__ float red[32];
  int t = blockIdx.x;
  int pos = tok_pos[t];
  size_t row = (size_t)t * ld;
  int QW = H * hd, KW = G * hd;
  float rq = 1.f, rk = 1.f;
  if (qw) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < QW; j += blockDim.x) { float v = ld_flag<A>(c, c_f32, row + j); ss += v * v; }
    rq = 1.0f / sqrtf(block_sum(ss, red) / (float)QW + eps);
  }
  if (kw && G > 0) {
    float ss = 0.f;
    for (int j = threadIdx.x; j < KW; j += blockDim.x) { float v = ld_flag<A>(c, c_f32, row + QW + j); ss += v * v; }
    rk = 1.0f / sqrtf(block_sum(ss, red) / (float)KW + eps);
  }
  size_t page_slot = 0;
  if (G > 0) {
    int page = block_table[(size_t)tok_seq[t] * max_pages + pos / SLLM_PAGE];
    page_slot = (size_t)page * G * SLLM_PAGE + (pos % SLLM_PAGE);       // + g * PAGE, times the head width
  }
  int half = rot >> 1;
  const float2* csr = cs + (size_t)pos * half;
  // the turning dims, a pair a thread
  for (int idx = threadIdx.x; idx < (H + G) * half; idx += blockDim.x) {
    int head = idx / half, i = idx % half;
    int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
    int col = head * hd;                                               // the key part follows the query part directly
    bool is_q = head < H;
    const void* w = is_q ? qw : kw;
    int wc = is_q ? col : col - QW;
    float r = is_q ? rq : rk;
    float x0 = ld_flag<A>(c, c_f32, row + col + i0) * r, x1 = ld_flag<A>(c, c_f32, row + col + i1) * r;
    if (w) { x0 *= load_w(w, w_f32, wc + i0); x1 *= load_w(w, w_f32, wc + i1); }
    float2 a = csr[i];
    float r0 = x0 * a.x - x1 * a.y, r1 = x1 * a.x + x0 * a.y;
    A* dst = is_q ? q_out + (size_t)t * ldq + col : kpages + (page_slot + (size_t)(head - H) * SLLM_PAGE) * hd;
    dst[i0] = from_f32<A>(r0);
    dst[i1] = from_f32<A>(r1);
  }
  // the dims that pass unturned
  int tail = hd - rot;
  for (int idx = threadIdx.x; idx < (H + G) * tail; idx += blockDim.x) {
    int head = idx / tail, j = rot + idx % tail;
    int col = head * hd;
    bool is_q = head < H;
    const void* w = is_q ? qw : kw;
    float x = ld_flag<A>(c, c_f32, row + col + j) * (is_q ? rq : rk);
    if (w) x *= load_w(w, w_f32, (is_q ? col : col - QW) + j);
    A* dst = is_q ? q_out + (size_t)t * ldq + col : kpages + (page_slot + (size_t)(head - H) * SLLM_PAGE) * hd;
    dst[j] = from_f32<A>(x);
  }
  // values as they are
  for (int idx = threadIdx.x; idx < G * vd; idx += blockDim.x) {
    int g = idx / vd, j = idx % vd;
    vpages[(page_slot + (size_t)g * SLLM_PAGE) * vd + j] = from_f32<A>(ld_flag<A>(c, c_f32, row + QW + KW + idx));
  }
}

// ------------------------------------------------------------------ a gate per head on the attention output
// o[t][h * vd + j] *= sigmoid(g[t * ldg + h]) (g float or A), one thread per element.
template <typename A>
__global__ void head_gate_kernel(A* __restrict__ o, int ldo, const void* __restrict__ g, int g_f32, int ldg, int T, int H, int vd) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t n = (size_t)T * H * vd;
  if (i >= n) return;
  int t = (int)(i / ((size_t)H * vd)), r = (int)(i % ((size_t)H * vd));
  float s = sigmoid_f(ld_flag<A>(g, g_f32, (size_t)t * ldg + r / vd));
  A* p = o + (size_t)t * ldo + r;
  *p = from_f32<A>(to_f32(*p) * s);
}

// ------------------------------------------------------------------ the stream takes its pending addend; a copy in A
// x float [n] += sum over p < P of d[p * n + i] (d float or A; P == 0: nothing to add); xb[i] = A(x[i]).
template <typename A>
__global__ void add_cast_kernel(float* __restrict__ x, const void* __restrict__ d, int d_f32, int P, A* __restrict__ xb, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i];
  for (int p = 0; p < P; p++) v += ld_flag<A>(d, d_f32, (size_t)p * n + i);
  if (P > 0) x[i] = v;
  xb[i] = from_f32<A>(v);
}

// ------------------------------------------------------------------ gelu(a) * a slice of the token's table row
// out[t][j] = gelu_tanh(a[t][j]) * table[ids[t]][col0 + j], j < D; table [rows][ldt] of A.
template <typename A>
__global__ void gelu_mul_rows_kernel(const A* __restrict__ a, int lda, const int* __restrict__ ids, const A* __restrict__ table,
                                     int ldt, int col0, A* __restrict__ out, int T, int D) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)T * D) return;
  int t = (int)(i / D), j = (int)(i % D);
  float e = to_f32(table[(size_t)ids[t] * ldt + col0 + j]);
  out[i] = from_f32<A>(gelu_tanh_f(to_f32(a[(size_t)t * lda + j])) * e);
}

// ------------------------------------------------------------------ x += y / rms(y) * w
// y float or A: [P][T][d] partial sums added in their order; a block per row, the row's y kept in shared memory.
template <typename A>
__global__ void add_rms_normed_kernel(float* __restrict__ x, const void* __restrict__ y, int y_f32, int P, int T,
                                      const void* __restrict__ w, int w_f32, int d, float eps) {
  extern __shared__ __align__(16) float rowbuf[];
  __shared__ float red[32];
  int t = blockIdx.x;
  float ss = 0.f;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float v = 0.f;
    for (int p = 0; p < P; p++) v += ld_flag<A>(y, y_f32, ((size_t)p * T + t) * d + j);
    rowbuf[j] = v;
    ss += v * v;
  }
  float r = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  for (int j = threadIdx.x; j < d; j += blockDim.x) x[(size_t)t * d + j] += rowbuf[j] * r * load_w(w, w_f32, j);
}

// ------------------------------------------------------------------ cap * tanh(x / cap)
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace gate
