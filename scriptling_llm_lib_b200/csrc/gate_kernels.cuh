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

// ------------------------------------------------------------------ convolution, norm, rotation, cache write
// The same as qk_norm_store behind a short causal convolution, one block a token and the row never leaving the
// chip: row t of y (A, row stride ldy) is the projection [queries | keys | values] of C = (H + G) hd + G vd
// columns; c[t][ch] = sum_j cw[ch][j] * y[t - taps + 1 + j][ch], rows before the step's first one of the sequence
// coming from its state [slot][taps - 1][C] (float, oldest first). c is kept as floats in shared memory, the sums
// of squares are taken on the way, then norm, rotation and stores as above. `own_state`: every sequence has one
// row in the step, and the block moves the sequence's state on by itself (a channel's entries are read and
// written by one thread); otherwise conv_state_kernel follows.
struct ConvNormArgs {
  const void* y; int ldy;
  const void* cw; int cw_f32; int taps;
  float* state; const int* seq_start; const int* tok_seq; const int* slots; int own_state;
  void* q_out; int ldq;
  const int* tok_pos; const int* block_table; int max_pages; const float2* cs;
  void* kpages; void* vpages;
  int H, G, hd, vd, rot, interleaved;
  const void* qw; const void* kw; int w_f32; float eps;
};

__device__ __forceinline__ void st2(float* p, float a, float b) { *(float2*)p = make_float2(a, b); }
__device__ __forceinline__ void st2(bf16* p, float a, float b) { *(__nv_bfloat162*)p = __floats2bfloat162_rn(a, b); }

template <typename A> __device__ __forceinline__ float4 ld4f(const void* p, int is_f32, size_t i) {
  return is_f32 ? ld4((const float*)p + i) : ld4((const A*)p + i);
}

// Four channels from c on with a number of taps known to the compiler: every load is issued before the first sum.
template <typename A, int TAPS>
__device__ __forceinline__ float4 conv_four(const ConvNormArgs& p, const A* __restrict__ y, float* st, int t, int first, int C, int c) {
  constexpr int HIST = TAPS - 1;
  float4 v[TAPS];
  float w[4 * TAPS];                           // the four channels' taps lie one behind the other
#pragma unroll
  for (int j = 0; j < TAPS; j++) {
    int s = t - HIST + j;
    v[j] = s >= first ? ld4(y + (size_t)s * p.ldy + c) : *(const float4*)(st + (size_t)(HIST + (s - first)) * C + c);
  }
#pragma unroll
  for (int m = 0; m < TAPS; m++) {
    float4 q = ld4f<A>(p.cw, p.cw_f32, (size_t)c * TAPS + 4 * m);
    w[4 * m] = q.x; w[4 * m + 1] = q.y; w[4 * m + 2] = q.z; w[4 * m + 3] = q.w;
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int j = 0; j < TAPS; j++) {
    acc.x += w[j] * v[j].x;
    acc.y += w[TAPS + j] * v[j].y;
    acc.z += w[2 * TAPS + j] * v[j].z;
    acc.w += w[3 * TAPS + j] * v[j].w;
  }
  if (p.own_state) {
#pragma unroll
    for (int j = 1; j < TAPS; j++) *(float4*)(st + (size_t)(j - 1) * C + c) = v[j];
  }
  return acc;
}

// VEC: four channels a thread. TAPS: the number of taps where the compiler knows it (VEC only), 0: p.taps.
template <typename A, int VEC, int TAPS>
__global__ void __launch_bounds__(256, 5) conv_qk_norm_store_kernel(ConvNormArgs p) {
  extern __shared__ __align__(16) float crow[];
  __shared__ float red[32];
  const A* y = (const A*)p.y;
  int t = blockIdx.x;
  int b = p.tok_seq[t];                        // the row's indices first, all at once: the stores below keep loads behind them
  int pos = p.tok_pos[t];
  int first = p.seq_start[b];
  int slot = p.slots[b];
  int page = p.G > 0 ? p.block_table[(size_t)b * p.max_pages + pos / SLLM_PAGE] : 0;
  int hist = p.taps - 1;
  int QW = p.H * p.hd, KW = p.G * p.hd, C = QW + KW + p.G * p.vd;
  float* st = p.state + (size_t)slot * hist * C;
  float ssq = 0.f, ssk = 0.f;
  if (VEC) {                                   // four channels a thread: C, QW, KW, ldy multiples of four
    for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (TAPS > 0) acc = conv_four<A, TAPS ? TAPS : 1>(p, y, st, t, first, C, c);
      else
      for (int j = 0; j < p.taps; j++) {
        int s = t - hist + j;
        float4 v = s >= first ? ld4(y + (size_t)s * p.ldy + c) : *(const float4*)(st + (size_t)(hist + (s - first)) * C + c);
        acc.x += load_w(p.cw, p.cw_f32, (size_t)c * p.taps + j) * v.x;
        acc.y += load_w(p.cw, p.cw_f32, (size_t)(c + 1) * p.taps + j) * v.y;
        acc.z += load_w(p.cw, p.cw_f32, (size_t)(c + 2) * p.taps + j) * v.z;
        acc.w += load_w(p.cw, p.cw_f32, (size_t)(c + 3) * p.taps + j) * v.w;
        if (p.own_state && j > 0) *(float4*)(st + (size_t)(j - 1) * C + c) = v;      // entry j moves to j - 1
      }
      *(float4*)(crow + c) = acc;
      float q = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
      if (c < QW) ssq += q; else if (c < QW + KW) ssk += q;
    }
  } else {
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float acc = 0.f;
      for (int j = 0; j < p.taps; j++) {
        int s = t - hist + j;
        float v = s >= first ? to_f32(y[(size_t)s * p.ldy + c]) : st[(size_t)(hist + (s - first)) * C + c];
        acc += load_w(p.cw, p.cw_f32, (size_t)c * p.taps + j) * v;
        if (p.own_state && j > 0) st[(size_t)(j - 1) * C + c] = v;
      }
      crow[c] = acc;
      if (c < QW) ssq += acc * acc; else if (c < QW + KW) ssk += acc * acc;
    }
  }
  float rq = 1.f, rk = 1.f;
  if (p.qw) rq = 1.0f / sqrtf(block_sum(ssq, red) / (float)QW + p.eps);
  if (p.kw && p.G > 0) rk = 1.0f / sqrtf(block_sum(ssk, red) / (float)KW + p.eps);
  __syncthreads();
  size_t page_slot = (size_t)page * p.G * SLLM_PAGE + (pos % SLLM_PAGE);
  A* q_row = (A*)p.q_out + (size_t)t * p.ldq;
  A* kp = (A*)p.kpages;
  A* vp = (A*)p.vpages;
  int hd = p.hd, half = p.rot >> 1;
  const float2* csr = p.cs + (size_t)pos * half;
  if (VEC && (p.interleaved || !(half & 1))) {
    // a warp a head, a lane two neighbouring dims (both in the same half of the turning part, or a pair of their own,
    // or behind it) and one store for both: no division on the way
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int head = wid; head < p.H + p.G; head += nw) {
      int col = head * hd;
      bool is_q = head < p.H;
      const void* w = is_q ? p.qw : p.kw;
      int wc = is_q ? col : col - QW;
      float r = is_q ? rq : rk;
      A* dst = is_q ? q_row + col : kp + (page_slot + (size_t)(head - p.H) * SLLM_PAGE) * hd;
      for (int d = 2 * lane; d < hd; d += 64) {
        float2 x = *(const float2*)(crow + col + d);
        float w0 = 1.f, w1 = 1.f;
        if (w) { w0 = load_w(w, p.w_f32, wc + d); w1 = load_w(w, p.w_f32, wc + d + 1); }
        float o0 = x.x * r * w0, o1 = x.y * r * w1;
        if (d < p.rot) {
          if (p.interleaved) {
            float2 a = csr[d >> 1];
            float t0 = o0 * a.x - o1 * a.y;
            o1 = o1 * a.x + o0 * a.y;
            o0 = t0;
          } else {
            bool low = d < half;
            int pd = low ? d + half : d - half;                        // the partner dims
            float2 y = *(const float2*)(crow + col + pd);
            float v0 = 1.f, v1 = 1.f;
            if (w) { v0 = load_w(w, p.w_f32, wc + pd); v1 = load_w(w, p.w_f32, wc + pd + 1); }
            float p0 = y.x * r * v0, p1 = y.y * r * v1;
            int ci = low ? d : pd;
            float2 a = csr[ci], bb = csr[ci + 1];
            o0 = low ? o0 * a.x - p0 * a.y : o0 * a.x + p0 * a.y;
            o1 = low ? o1 * bb.x - p1 * bb.y : o1 * bb.x + p1 * bb.y;
          }
        }
        st2(dst + d, o0, o1);
      }
    }
    for (int g = wid; g < p.G; g += nw)
      for (int j = 4 * lane; j < p.vd; j += 128)
        st4(vp + (page_slot + (size_t)g * SLLM_PAGE) * p.vd + j, *(const float4*)(crow + QW + KW + g * p.vd + j));
    return;
  }
  for (int idx = threadIdx.x; idx < (p.H + p.G) * half; idx += blockDim.x) {
    int head = idx / half, i = idx % half;
    int i0 = p.interleaved ? 2 * i : i, i1 = p.interleaved ? 2 * i + 1 : i + half;
    int col = head * hd;
    bool is_q = head < p.H;
    const void* w = is_q ? p.qw : p.kw;
    int wc = is_q ? col : col - QW;
    float r = is_q ? rq : rk;
    float x0 = crow[col + i0] * r, x1 = crow[col + i1] * r;
    if (w) { x0 *= load_w(w, p.w_f32, wc + i0); x1 *= load_w(w, p.w_f32, wc + i1); }
    float2 a = csr[i];
    A* dst = is_q ? q_row + col : kp + (page_slot + (size_t)(head - p.H) * SLLM_PAGE) * hd;
    dst[i0] = from_f32<A>(x0 * a.x - x1 * a.y);
    dst[i1] = from_f32<A>(x1 * a.x + x0 * a.y);
  }
  int tail = hd - p.rot;
  for (int idx = threadIdx.x; idx < (p.H + p.G) * tail; idx += blockDim.x) {
    int head = idx / tail, j = p.rot + idx % tail;
    int col = head * hd;
    bool is_q = head < p.H;
    const void* w = is_q ? p.qw : p.kw;
    float x = crow[col + j] * (is_q ? rq : rk);
    if (w) x *= load_w(w, p.w_f32, (is_q ? col : col - QW) + j);
    A* dst = is_q ? q_row + col : kp + (page_slot + (size_t)(head - p.H) * SLLM_PAGE) * hd;
    dst[j] = from_f32<A>(x);
  }
  for (int idx = threadIdx.x; idx < p.G * p.vd; idx += blockDim.x) {
    int g = idx / p.vd, j = idx % p.vd;
    vp[(page_slot + (size_t)g * SLLM_PAGE) * p.vd + j] = from_f32<A>(crow[QW + KW + idx]);
  }
}

// After a step of several rows a sequence: the state becomes the last taps - 1 rows of [state | the step's rows].
template <typename A>
__global__ void conv_state_kernel(ConvNormArgs p, int n_seqs, int C) {
  int b = blockIdx.x;
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C || b >= n_seqs) return;
  const A* y = (const A*)p.y;
  int first = p.seq_start[b], n = p.seq_start[b + 1] - first;
  int hist = p.taps - 1;
  float* st = p.state + (size_t)p.slots[b] * hist * C;
  for (int k = 0; k < hist; k++) {              // ascending: a kept entry moves down before its place is written
    int s = n + k - hist;                       // a row of the step, or (negative) an entry of the old state
    st[(size_t)k * C + c] = s >= 0 ? to_f32(y[(size_t)(first + s) * p.ldy + c]) : st[(size_t)(hist + s) * C + c];
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

// eight neighbouring columns a thread: vd, ldo multiples of eight, o aligned for the wide access
template <typename A>
__global__ void head_gate_vec8_kernel(A* __restrict__ o, int ldo, const void* __restrict__ g, int g_f32, int ldg, int T, int H, int vd) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  size_t wrow = (size_t)H * vd;
  if (i >= (size_t)T * wrow) return;
  int t = (int)(i / wrow), r = (int)(i % wrow);
  float s = sigmoid_f(ld_flag<A>(g, g_f32, (size_t)t * ldg + r / vd));
  A* p = o + (size_t)t * ldo + r;
  F8 v = ld8(p);
#pragma unroll
  for (int k = 0; k < 8; k++) v.f[k] *= s;
  st8(p, v);
}

// four neighbouring columns a thread: vd, ldo multiples of four, o aligned for the wide access
template <typename A>
__global__ void head_gate_vec_kernel(A* __restrict__ o, int ldo, const void* __restrict__ g, int g_f32, int ldg, int T, int H, int vd) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  size_t wrow = (size_t)H * vd;
  if (i >= (size_t)T * wrow) return;
  int t = (int)(i / wrow), r = (int)(i % wrow);
  float s = sigmoid_f(ld_flag<A>(g, g_f32, (size_t)t * ldg + r / vd));
  A* p = o + (size_t)t * ldo + r;
  float4 v = ld4(p);
  st4(p, make_float4(v.x * s, v.y * s, v.z * s, v.w * s));
}

// a logit per element (vd == 1), eight neighbouring columns a thread: o[t][j] *= sigmoid(g[t][j]), g of the element type;
// n, ldo, ldg multiples of eight, both aligned for the wide access
template <typename A>
__global__ void elem_gate_vec8_kernel(A* __restrict__ o, int ldo, const A* __restrict__ g, int ldg, int T, int n) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= (size_t)T * n) return;
  int t = (int)(i / n), r = (int)(i % n);
  A* p = o + (size_t)t * ldo + r;
  F8 v = ld8(p), w = ld8(g + (size_t)t * ldg + r);
#pragma unroll
  for (int k = 0; k < 8; k++) v.f[k] *= sigmoid_f(w.f[k]);
  st8(p, v);
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

// four elements a thread (n a multiple of four)
template <typename A>
__global__ void add_cast_vec_kernel(float* __restrict__ x, const void* __restrict__ d, int d_f32, int P, A* __restrict__ xb, size_t n) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 v = *(const float4*)(x + i);
  for (int p = 0; p < P; p++) {
    float4 a = ld4f<A>(d, d_f32, (size_t)p * n + i);
    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
  }
  if (P > 0) *(float4*)(x + i) = v;
  st4(xb + i, v);
}

// several addends at once: x float [T][d] += sum over the list's entries k, each [P_k][T][d] partial sums (float or A) added in
// their order, and + vec[j] (float [d], or null) on every row; xb (A, or null) = the rounded stream. One pass over the stream.
#define GATE_MAX_ADDENDS 8
struct AddList {
  const void* p[GATE_MAX_ADDENDS];
  int f32[GATE_MAX_ADDENDS];
  int P[GATE_MAX_ADDENDS];
  int count;
};
template <typename A>
__global__ void add_list_cast_kernel(float* __restrict__ x, AddList l, const float* __restrict__ vec, int d, A* __restrict__ xb, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i];
  for (int k = 0; k < l.count; k++)
    for (int q = 0; q < l.P[k]; q++) v += ld_flag<A>(l.p[k], l.f32[k], (size_t)q * n + i);
  if (vec) v += vec[i % d];
  x[i] = v;
  if (xb) xb[i] = from_f32<A>(v);
}
template <typename A>
__global__ void add_list_cast_vec_kernel(float* __restrict__ x, AddList l, const float* __restrict__ vec, int d, A* __restrict__ xb, size_t n) {
  size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 v = *(const float4*)(x + i);
  for (int k = 0; k < l.count; k++)
    for (int q = 0; q < l.P[k]; q++) {
      float4 a = ld4f<A>(l.p[k], l.f32[k], (size_t)q * n + i);
      v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
    }
  if (vec) {
    float4 b = *(const float4*)(vec + i % d);
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  *(float4*)(x + i) = v;
  if (xb) st4(xb + i, v);
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
// With `out` (A, [gridDim.x][d]) the row's norm for the next reader follows in the same pass: out = x / rms(x) * w2 of
// the stream as it now stands, or with `b2` the norm without statistics tanh(alpha2 x) * w2 + b2 (w2, b2 float then);
// `rows` (or null) picks the stream's rows that are worked on, out's rows stay in order. `vec` (float [d], or null)
// is added to the row as well.
template <typename A>
__global__ void add_rms_normed_kernel(float* __restrict__ x, const void* __restrict__ y, int y_f32, int P, int T,
                                      const void* __restrict__ w, int w_f32, int d, float eps, const int* __restrict__ rows,
                                      const void* __restrict__ w2, int w2_f32, float eps2, A* __restrict__ out,
                                      const float* __restrict__ vec, const float* __restrict__ b2, float alpha2) {
  extern __shared__ __align__(16) float rowbuf[];
  __shared__ float red[32];
  int t = rows ? rows[blockIdx.x] : blockIdx.x;
  float ss = 0.f;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float v = 0.f;
    for (int p = 0; p < P; p++) v += ld_flag<A>(y, y_f32, ((size_t)p * T + t) * d + j);
    rowbuf[j] = v;
    ss += v * v;
  }
  float r = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  float ss2 = 0.f;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float v = x[(size_t)t * d + j] + rowbuf[j] * r * load_w(w, w_f32, j);
    if (vec) v += vec[j];
    x[(size_t)t * d + j] = v;
    rowbuf[j] = v;                             // a column is one thread's in every pass
    ss2 += v * v;
  }
  if (!out) return;
  if (b2) {
    for (int j = threadIdx.x; j < d; j += blockDim.x)
      out[(size_t)blockIdx.x * d + j] = from_f32<A>(tanhf(alpha2 * rowbuf[j]) * load_w(w2, 1, j) + b2[j]);
    return;
  }
  float r2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)d + eps2);
  for (int j = threadIdx.x; j < d; j += blockDim.x)
    out[(size_t)blockIdx.x * d + j] = from_f32<A>(rowbuf[j] * r2 * load_w(w2, w2_f32, j));
}

// four columns a thread (d a multiple of four); the partial sums are added in the same order
template <typename A>
__global__ void add_rms_normed_vec_kernel(float* __restrict__ x, const void* __restrict__ y, int y_f32, int P, int T,
                                          const void* __restrict__ w, int w_f32, int d, float eps, const int* __restrict__ rows,
                                          const void* __restrict__ w2, int w2_f32, float eps2, A* __restrict__ out,
                                          const float* __restrict__ vec, const float* __restrict__ b2, float alpha2) {
  extern __shared__ __align__(16) float rowbuf[];
  __shared__ float red[32];
  int t = rows ? rows[blockIdx.x] : blockIdx.x;
  float ss = 0.f;
  for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < P; p++) {
      float4 a = ld4f<A>(y, y_f32, ((size_t)p * T + t) * d + j);
      v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
    }
    *(float4*)(rowbuf + j) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  float r = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
  float ss2 = 0.f;
  for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
    float4 v = *(const float4*)(rowbuf + j);
    float4 xv = *(const float4*)(x + (size_t)t * d + j);
    xv.x += v.x * r * load_w(w, w_f32, j);
    xv.y += v.y * r * load_w(w, w_f32, j + 1);
    xv.z += v.z * r * load_w(w, w_f32, j + 2);
    xv.w += v.w * r * load_w(w, w_f32, j + 3);
    if (vec) {
      float4 b = *(const float4*)(vec + j);
      xv.x += b.x; xv.y += b.y; xv.z += b.z; xv.w += b.w;
    }
    *(float4*)(x + (size_t)t * d + j) = xv;
    *(float4*)(rowbuf + j) = xv;
    ss2 += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
  }
  if (!out) return;
  if (b2) {
    for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
      float4 v = *(const float4*)(rowbuf + j);
      float4 ww = *(const float4*)((const float*)w2 + j), bb = *(const float4*)(b2 + j);
      st4(out + (size_t)blockIdx.x * d + j, make_float4(tanhf(alpha2 * v.x) * ww.x + bb.x, tanhf(alpha2 * v.y) * ww.y + bb.y,
                                                        tanhf(alpha2 * v.z) * ww.z + bb.z, tanhf(alpha2 * v.w) * ww.w + bb.w));
    }
    return;
  }
  float r2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)d + eps2);
  for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
    float4 v = *(const float4*)(rowbuf + j);
    st4(out + (size_t)blockIdx.x * d + j, make_float4(v.x * r2 * load_w(w2, w2_f32, j), v.y * r2 * load_w(w2, w2_f32, j + 1),
                                                      v.z * r2 * load_w(w2, w2_f32, j + 2), v.w * r2 * load_w(w2, w2_f32, j + 3)));
  }
}

// ------------------------------------------------------------------ cap * tanh(x * scale / cap) (cap <= 0: x * scale)
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float scale) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = x[i] * scale;
  x[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

}  // namespace gate
