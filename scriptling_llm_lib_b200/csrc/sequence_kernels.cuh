// Kernels of the mixers that carry state along a sequence, and of what stands around them: a norm
// that takes several weighted addends and may subtract the mean, a short causal convolution over
// time with its last inputs kept per sequence, the gated delta rule, a gated linear recurrence with
// block-diagonal gates, and attention whose keys and values have different widths.
//
// All of them work on the packed rows of a step (seq_start[b] .. seq_start[b + 1] are the rows of
// sequence b, in order of position) and find a sequence's state through slots[b]. What the state
// holds is float32 whatever the element type A of activations and weights; every sum, norm, gate,
// decay and softmax here is float32 too. A buffer whose precision depends on its place in the model
// (a projection's output in A, a norm's output in float) is passed as void* with a flag.
#pragma once
#include "common.cuh"

template <typename A> __device__ __forceinline__ float ld_flag(const void* p, int is_f32, size_t i) {
  return is_f32 ? ((const float*)p)[i] : to_f32(((const A*)p)[i]);
}
template <typename A> __device__ __forceinline__ void st_flag(void* p, int is_f32, size_t i, float v) {
  if (is_f32) ((float*)p)[i] = v;
  else ((A*)p)[i] = from_f32<A>(v);
}
template <typename A> __device__ __forceinline__ float4 ld4_flag(const void* p, int is_f32, size_t i) {
  return is_f32 ? ld4((const float*)p + i) : ld4((const A*)p + i);
}
template <typename A> __device__ __forceinline__ void st4_flag(void* p, int is_f32, size_t i, float4 v) {
  if (is_f32) st4((float*)p + i, v);
  else st4((A*)p + i, v);
}
__device__ __forceinline__ float4 ld4_w(const void* w, int is_f32, size_t i) {
  return is_f32 ? ld4((const float*)w + i) : ld4((const bf16*)w + i);
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------ residual sum + norm
// v = x[row] + sum_a coef[a] * addend[a][row]; center: y = (v - mean) / sqrt(var + eps) * w with var the mean of
// the squared deviations; else y = v / sqrt(mean(v^2) + eps) * w. rows == nullptr: x is updated in place.
#define SEQ_MAX_ADDENDS 16
struct SeqAddends {
  const void* p[SEQ_MAX_ADDENDS];
  float coef[SEQ_MAX_ADDENDS];
  int is_f32[SEQ_MAX_ADDENDS];
  int n;
};

template <typename A>
__global__ void add_norm_kernel(float* __restrict__ x, SeqAddends ad, const int* __restrict__ rows,
                                const void* __restrict__ w, int w_f32, void* __restrict__ y, int y_f32, int d, float eps,
                                int center, int vec) {
  extern __shared__ __align__(16) float sm_row[];
  __shared__ float red[32];
  int r = blockIdx.x;
  size_t in = rows ? (size_t)rows[r] : (size_t)r;
  float* xr = x + in * d;
  bool update = rows == nullptr && ad.n > 0;
  float s = 0.f;
  if (vec) {                                    // four elements per access: d, every row and the weight 16-byte aligned
    for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
      float4 v = *(const float4*)(xr + j);
      for (int a = 0; a < ad.n; a++) {
        float4 t = ld4_flag<A>(ad.p[a], ad.is_f32[a], in * d + j);
        float c = ad.coef[a];
        v.x += c * t.x; v.y += c * t.y; v.z += c * t.z; v.w += c * t.w;
      }
      *(float4*)(sm_row + j) = v;
      if (update) *(float4*)(xr + j) = v;
      s += (v.x + v.y) + (v.z + v.w);
    }
    float mean = 0.f;
    if (center) mean = block_sum(s, red) / (float)d;
    float ss = 0.f;
    for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
      float4 v = *(const float4*)(sm_row + j);
      float a = v.x - mean, b = v.y - mean, c = v.z - mean, e = v.w - mean;
      ss += (a * a + b * b) + (c * c + e * e);
    }
    ss = block_sum(ss, red);
    float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
      float4 v = *(const float4*)(sm_row + j);
      float4 wv = ld4_w(w, w_f32, j);
      st4_flag<A>(y, y_f32, (size_t)r * d + j, make_float4(((v.x - mean) * inv) * wv.x, ((v.y - mean) * inv) * wv.y,
                                                            ((v.z - mean) * inv) * wv.z, ((v.w - mean) * inv) * wv.w));
    }
    return;
  }
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float v = xr[j];
    for (int a = 0; a < ad.n; a++) v += ad.coef[a] * ld_flag<A>(ad.p[a], ad.is_f32[a], in * d + j);
    sm_row[j] = v;
    if (update) xr[j] = v;
    s += v;
  }
  float mean = 0.f;
  if (center) mean = block_sum(s, red) / (float)d;
  float ss = 0.f;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float c = sm_row[j] - mean;
    ss += c * c;
  }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)d + eps);
  for (int j = threadIdx.x; j < d; j += blockDim.x)
    st_flag<A>(y, y_f32, (size_t)r * d + j, ((sm_row[j] - mean) * inv) * load_w(w, w_f32, j));
}

// ------------------------------------------------------------------ short causal convolution over time
// in(t)[c] = x[t][c] + in_bias[c]; y[t][c] = sum_j w[c][j] * in(t - taps + 1 + j)[c] + out_bias[c] (+ in(t)[c] when
// add_input), then the activation (0 none, 1 silu). Inputs before the step's first row come from the
// sequence's state [slot][taps - 1][C] (oldest first; zero for a new sequence). y2 (or null): the same
// values once more in the element type.
struct ConvArgs {
  const void* x; int x_f32; int ldx;
  const void* w; int w_f32;
  const void* in_bias; const void* out_bias; int b_f32;
  float* state;
  const int* seq_start; const int* tok_seq; const int* slots;
  void* y; int y_f32; int ldy;
  void* y2; int ldy2;
  int C, taps, add_input, act;
};

template <typename A>
__global__ void causal_conv_kernel(ConvArgs p) {
  int t = blockIdx.x;
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  int b = p.tok_seq[t];
  int first = p.seq_start[b];
  int hist = p.taps - 1;
  const float* st = p.state + (size_t)p.slots[b] * hist * p.C;
  float ib = p.in_bias ? load_w(p.in_bias, p.b_f32, c) : 0.f;
  float acc = 0.f, cur = 0.f;
  for (int j = 0; j < p.taps; j++) {
    int s = t - hist + j;                       // the row this tap reads
    float v;
    if (s >= first) v = ld_flag<A>(p.x, p.x_f32, (size_t)s * p.ldx + c) + ib;
    else v = st[(size_t)(hist + (s - first)) * p.C + c];      // s - first in [-hist, -1]
    acc += load_w(p.w, p.w_f32, (size_t)c * p.taps + j) * v;
    cur = v;
  }
  if (p.out_bias) acc += load_w(p.out_bias, p.b_f32, c);
  if (p.add_input) acc += cur;
  if (p.act == 1) acc = silu_f(acc);
  st_flag<A>(p.y, p.y_f32, (size_t)t * p.ldy + c, acc);
  if (p.y2) ((A*)p.y2)[(size_t)t * p.ldy2 + c] = from_f32<A>(acc);
}

// The same, four neighbouring channels per thread with 16-byte (float) or 8-byte accesses: C, the row strides
// and the buffers' starts are multiples of four elements.
template <typename A>
__global__ void causal_conv_vec_kernel(ConvArgs p) {
  int t = blockIdx.x;
  int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= p.C) return;
  int b = p.tok_seq[t];
  int first = p.seq_start[b];
  int hist = p.taps - 1;
  const float* st = p.state + (size_t)p.slots[b] * hist * p.C;
  float4 ib = p.in_bias ? ld4_w(p.in_bias, p.b_f32, c) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), cur = acc;
  for (int j = 0; j < p.taps; j++) {
    int s = t - hist + j;
    float4 v;
    if (s >= first) {
      v = ld4_flag<A>(p.x, p.x_f32, (size_t)s * p.ldx + c);
      v.x += ib.x; v.y += ib.y; v.z += ib.z; v.w += ib.w;
    } else {
      v = *(const float4*)(st + (size_t)(hist + (s - first)) * p.C + c);
    }
    acc.x += load_w(p.w, p.w_f32, (size_t)c * p.taps + j) * v.x;
    acc.y += load_w(p.w, p.w_f32, (size_t)(c + 1) * p.taps + j) * v.y;
    acc.z += load_w(p.w, p.w_f32, (size_t)(c + 2) * p.taps + j) * v.z;
    acc.w += load_w(p.w, p.w_f32, (size_t)(c + 3) * p.taps + j) * v.w;
    cur = v;
  }
  if (p.out_bias) {
    float4 ob = ld4_w(p.out_bias, p.b_f32, c);
    acc.x += ob.x; acc.y += ob.y; acc.z += ob.z; acc.w += ob.w;
  }
  if (p.add_input) { acc.x += cur.x; acc.y += cur.y; acc.z += cur.z; acc.w += cur.w; }
  if (p.act == 1) { acc.x = silu_f(acc.x); acc.y = silu_f(acc.y); acc.z = silu_f(acc.z); acc.w = silu_f(acc.w); }
  st4_flag<A>(p.y, p.y_f32, (size_t)t * p.ldy + c, acc);
  if (p.y2) st4((A*)p.y2 + (size_t)t * p.ldy2 + c, acc);
}

// After the convolution of a step: the state becomes the last taps - 1 inputs of [state | step's rows].
template <typename A>
__global__ void conv_state_update_kernel(ConvArgs p, int n_seqs) {
  int b = blockIdx.x;
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.C || b >= n_seqs) return;
  int first = p.seq_start[b], n = p.seq_start[b + 1] - first;
  int hist = p.taps - 1;
  float* st = p.state + (size_t)p.slots[b] * hist * p.C;
  float ib = p.in_bias ? load_w(p.in_bias, p.b_f32, c) : 0.f;
  for (int k = 0; k < hist; k++) {              // ascending: a kept entry moves down before its place is written
    int s = n + k - hist;                       // row of the step, or (negative) an entry of the old state
    float v = s >= 0 ? ld_flag<A>(p.x, p.x_f32, (size_t)(first + s) * p.ldx + c) + ib : st[(size_t)(hist + s) * p.C + c];
    st[(size_t)k * p.C + c] = v;
  }
}

// ------------------------------------------------------------------ positions, value norm, cache write
// Row t of qkv holds [H query heads of hd | G key heads of hd | G value heads of vd]. The first `rot` dims of
// every query and key head are turned by the token's position (table cs[pos][i] = (cos, sin)); queries are
// rewritten in place, keys go to the token's place in the paged cache. Values are divided by their root mean
// square over vd (v_eps >= 0; v_eps < 0: stored as they are) and stored beside them. G == 0: queries only.
template <typename A>
__global__ void kv_store_kernel(A* __restrict__ qkv, int ld, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                const int* __restrict__ block_table, int max_pages, const float2* __restrict__ cs,
                                A* __restrict__ kpages, A* __restrict__ vpages, int H, int G, int hd, int vd, int rot,
                                int interleaved, float v_eps) {
  int t = blockIdx.x;
  int pos = tok_pos[t];
  int half = rot >> 1;
  A* row = qkv + (size_t)t * ld;
  size_t page_slot = 0;
  if (G > 0) {
    int page = block_table[(size_t)tok_seq[t] * max_pages + pos / SLLM_PAGE];
    page_slot = (size_t)page * G * SLLM_PAGE + (pos % SLLM_PAGE);       // + g * PAGE, times the head width
  }
  const float2* csr = cs + (size_t)pos * half;
  for (int idx = threadIdx.x; idx < (H + G) * half; idx += blockDim.x) {
    int head = idx / half, i = idx % half;
    int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
    A* h = row + (size_t)head * hd;
    float x0 = to_f32(h[i0]), x1 = to_f32(h[i1]);
    float2 c = csr[i];
    float r0 = x0 * c.x - x1 * c.y, r1 = x1 * c.x + x0 * c.y;
    if (head < H) {
      h[i0] = from_f32<A>(r0);
      h[i1] = from_f32<A>(r1);
    } else {
      A* dst = kpages + (page_slot + (size_t)(head - H) * SLLM_PAGE) * hd;
      dst[i0] = from_f32<A>(r0);
      dst[i1] = from_f32<A>(r1);
    }
  }
  if (G == 0) return;
  int tail = hd - rot;
  for (int idx = threadIdx.x; idx < G * tail; idx += blockDim.x) {
    int g = idx / tail, j = rot + idx % tail;
    kpages[(page_slot + (size_t)g * SLLM_PAGE) * hd + j] = row[(size_t)(H + g) * hd + j];
  }
  // values: a warp per head
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const A* vrow = row + (size_t)(H + G) * hd;
  for (int g = wid; g < G; g += nw) {
    float scale = 1.f;
    if (v_eps >= 0.f) {
      float ss = 0.f;
      for (int j = lane; j < vd; j += 32) {
        float v = to_f32(vrow[(size_t)g * vd + j]);
        ss += v * v;
      }
      ss = warp_sum(ss);
      scale = 1.0f / sqrtf(ss / (float)vd + v_eps);
    }
    A* dst = vpages + (page_slot + (size_t)g * SLLM_PAGE) * vd;
    for (int j = lane; j < vd; j += 32) dst[j] = from_f32<A>(to_f32(vrow[(size_t)g * vd + j]) * scale);
  }
}

// ------------------------------------------------------------------ attention, keys of width hd, values of width vd
// One warp per (row, query head), four to a block with the heads running fastest, so that the warps of a block
// mostly read the same key/value head. The warp takes its visible keys 32 at a time: a lane scores one key (its
// row of the cache against the query in shared memory), the running maximum and sum of the softmax are updated
// once per 32 keys, and the weighted values are summed with a lane per value column (vd / 32 sums a lane), the
// weights passed round by shuffles. Row t sees the keys at positions max(0, pos - window + 1) .. pos of its own
// sequence (window 0: all of them). vec8: key rows can be read 8 elements (16 bytes of bfloat16, 32 of float) at a time.
// WPI warps per (row, head): 1, or 4 for steps of few rows (a decode step), where the four take every fourth
// group of 32 keys and are merged through shared memory at the end.
template <typename A, int NV, int WPI>
__global__ void __launch_bounds__(128) attn_wide_value_kernel(const A* __restrict__ q, int q_ld, A* __restrict__ out, int out_ld,
                                                              const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                                              const int* __restrict__ block_table, int max_pages,
                                                              const A* __restrict__ kpages, const A* __restrict__ vpages, int T,
                                                              int H, int G, int hd, int vd, int window, float scale, int vec8) {
  extern __shared__ __align__(16) float sm_att[];            // 4 / WPI queries of hd floats; WPI == 4: then 4 x (32 NV + 2) to merge
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  size_t item = (size_t)blockIdx.x * (4 / WPI) + wid / WPI;
  int sub = wid % WPI;
  bool have = item < (size_t)T * H;
  if (!have && WPI == 1) return;
  if (!have) item = (size_t)T * H - 1;          // WPI == 4: one item a block, so this does not happen; keeps the barrier whole
  int t = (int)(item / H), h = (int)(item % H);
  int g = h / (H / G);
  int pos = tok_pos[t];
  const int* pages = block_table + (size_t)tok_seq[t] * max_pages;
  float* qs = sm_att + (size_t)(wid / WPI) * hd;
  if (WPI == 1) {
    for (int j = lane; j < hd; j += 32) qs[j] = to_f32(q[(size_t)t * q_ld + (size_t)h * hd + j]) * scale;
    __syncwarp();
  } else {
    for (int j = threadIdx.x; j < hd; j += 128) qs[j] = to_f32(q[(size_t)t * q_ld + (size_t)h * hd + j]) * scale;
    __syncthreads();
  }
  int lo = first_seen(pos, window);
  float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) acc[i] = 0.f;
  for (int base = lo + 32 * sub; base <= pos; base += 32 * WPI) {
    int kp = base + lane;
    bool seen = kp <= pos;
    unsigned at = 0;                            // the key's row in the store: (page * G + g) * PAGE + offset
    float sc = -INFINITY;
    if (seen) {
      at = ((unsigned)pages[kp / SLLM_PAGE] * G + g) * SLLM_PAGE + (kp % SLLM_PAGE);
      const A* kr = kpages + (size_t)at * hd;
      float s0 = 0.f, s1 = 0.f;
      if (vec8) {
        for (int d = 0; d < hd; d += 8) {
          F8 kv = ld8(kr + d);
          s0 += qs[d] * kv.f[0] + qs[d + 2] * kv.f[2] + qs[d + 4] * kv.f[4] + qs[d + 6] * kv.f[6];
          s1 += qs[d + 1] * kv.f[1] + qs[d + 3] * kv.f[3] + qs[d + 5] * kv.f[5] + qs[d + 7] * kv.f[7];
        }
      } else {
        for (int d = 0; d < hd; d++) s0 += qs[d] * to_f32(kr[d]);
      }
      sc = s0 + s1;
    }
    float m_new = fmaxf(m, warp_max(sc));
    float c = expf(m - m_new);                  // expf(-inf) = 0 before the first key
    float pw = seen ? expf(sc - m_new) : 0.f;
    l = l * c + warp_sum(pw);
#pragma unroll
    for (int i = 0; i < NV; i++) acc[i] *= c;
    int n = min(32, pos - base + 1);
    // UB keys' values asked for together, then summed: eight where few warps run (their loads must overlap one
    // another), one where the GPU is full of warps (registers are worth more there)
    constexpr int UB = WPI == 1 ? 1 : 8;
    for (int j0 = 0; j0 < n; j0 += UB) {
      float pj[UB], vals[UB][NV];
#pragma unroll
      for (int jj = 0; jj < UB; jj++) {
        int src = min(j0 + jj, n - 1);
        pj[jj] = j0 + jj < n ? __shfl_sync(0xffffffffu, pw, src) : 0.f;
        unsigned aj = __shfl_sync(0xffffffffu, at, src);
        const A* vr = vpages + (size_t)aj * vd;
#pragma unroll
        for (int i = 0; i < NV; i++) {
          int j = lane + 32 * i;
          vals[jj][i] = j < vd ? to_f32(vr[j]) : 0.f;
        }
      }
#pragma unroll
      for (int jj = 0; jj < UB; jj++) {
#pragma unroll
        for (int i = 0; i < NV; i++) acc[i] += pj[jj] * vals[jj][i];
      }
    }
    m = m_new;
  }
  if (WPI == 1) {
    float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      int j = lane + 32 * i;
      if (j < vd) out[(size_t)t * out_ld + (size_t)h * vd + j] = from_f32<A>(acc[i] * inv);
    }
    return;
  }
  float* part = sm_att + hd + (size_t)wid * (32 * NV + 2);
#pragma unroll
  for (int i = 0; i < NV; i++) part[lane + 32 * i] = acc[i];
  if (lane == 0) { part[32 * NV] = m; part[32 * NV + 1] = l; }
  __syncthreads();
  if (wid == 0 && have) {
    float M = -INFINITY;
    for (int w = 0; w < 4; w++) M = fmaxf(M, sm_att[hd + (size_t)w * (32 * NV + 2) + 32 * NV]);
    float L = 0.f, o[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) o[i] = 0.f;
    for (int w = 0; w < 4; w++) {               // fixed order
      const float* pa = sm_att + hd + (size_t)w * (32 * NV + 2);
      float mw = pa[32 * NV];
      if (mw == -INFINITY) continue;
      float c = expf(mw - M);
      L += pa[32 * NV + 1] * c;
#pragma unroll
      for (int i = 0; i < NV; i++) o[i] += pa[lane + 32 * i] * c;
    }
    float inv = 1.0f / L;
#pragma unroll
    for (int i = 0; i < NV; i++) {
      int j = lane + 32 * i;
      if (j < vd) out[(size_t)t * out_ld + (size_t)h * vd + j] = from_f32<A>(o[i] * inv);
    }
  }
}

// ------------------------------------------------------------------ gated delta rule
// Before the recurrence, per row: queries and keys (float, [G heads of dk] each, at qk and qk + G * dk of a row
// of ld_qk floats) become unit vectors x / sqrt(sum x^2 + 1e-6), queries times dk^-1/2; ba holds the raw
// projections [H betas | H decays] of a row (ld_ba floats): beta = sigmoid(b), decay = exp(-exp(A_log) *
// softplus(a + dt_bias)), written to bd[t][0..H) and bd[t][H..2H); bd[t][2H + g] receives k . q of q/k head g
// (after the scaling), which the recurrence's read-out needs. A row of bd has 2H + G floats.
template <typename A>
__global__ void delta_prepare_kernel(float* __restrict__ qk, int ld_qk, const float* __restrict__ ba, int ld_ba,
                                     const void* __restrict__ a_log, const void* __restrict__ dt_bias, int w_f32,
                                     float* __restrict__ bd, int H, int G, int dk) {
  int t = blockIdx.x;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float qmult = rsqrtf((float)dk);
  float* brow = bd + (size_t)t * (2 * H + G);
  for (int gg = wid; gg < G; gg += nw) {
    float* qv = qk + (size_t)t * ld_qk + (size_t)gg * dk;
    float* kv = qv + (size_t)G * dk;
    float sq = 0.f, sk = 0.f;
    for (int j = lane; j < dk; j += 32) { sq += qv[j] * qv[j]; sk += kv[j] * kv[j]; }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    float iq = qmult / sqrtf(sq + 1e-6f), ik = 1.0f / sqrtf(sk + 1e-6f);
    float kq = 0.f;
    for (int j = lane; j < dk; j += 32) {
      float a = qv[j] * iq, b2 = kv[j] * ik;
      qv[j] = a;
      kv[j] = b2;
      kq += a * b2;
    }
    kq = warp_sum(kq);
    if (lane == 0) brow[2 * H + gg] = kq;
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float* r = ba + (size_t)t * ld_ba;
    brow[h] = sigmoid_f(r[h]);
    float dt = softplus_f(r[H + h] + load_w(dt_bias, w_f32, h));
    brow[H + h] = expf(-expf(load_w(a_log, w_f32, h)) * dt);
  }
}

// The recurrence itself. A block of four computing warps per (8 value columns, head, sequence): DR_LPC = 16 lanes
// share a column j of the head's state S [dk][dv] (row-major in the state tensor [slot][H][dk][dv]); lane r of
// them keeps the rows 64 m + 4 r + (0..3), m = 0, 1, ..., in registers, and the block walks the sequence's rows in order:
//   S *= decay;  u = beta * (v_j - sum_d S[d] k[d]);  S[d] += k[d] u;  o_j = sum_d S[d] q[d].
// The read-out of the new state is taken from the old one, o_j = decay * sum_d S_old[d] q[d] + u * (k . q) with
// k . q from the prepare kernel, so both sums run side by side (each in four partial sums, ending with four
// shuffles among the sixteen lanes) and a row costs one round of shuffles, not two. What a row brings
// (q, k, the 8 values, beta, decay, k . q) comes through a ring of DR_RING rows in shared memory filled by
// asynchronous copies, a batch of DR_BATCH rows ahead of the batch worked on, so the walk waits for memory once, not
// once per row. A third warp does nothing but send the copies off, so that the computing warps' instructions are
// the sums alone; two block barriers per batch hand the ring's halves back and forth. DKR rows per lane (a multiple of 4): dk <= 16 DKR. vec: every copy
// is 16 bytes and aligned.
#define DR_NB 4            // batches in the ring
#define DR_DIRECT_MAX 4    // rows of a sequence in a step up to which the ring is not worth its set-up
#define DR_RING 32
#define DR_BATCH 8      // rows per barrier; two batches fill the ring
#ifndef DR_LPC
#define DR_LPC 16          // lanes that share a state column
#endif
#define DR_THREADS (8 * DR_LPC)     // computing threads: 8 columns x DR_LPC lanes
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DKR>
__global__ void __launch_bounds__(DR_THREADS + 32) delta_rule_kernel(const float* __restrict__ qk, int ld_qk,
                                                                      const float* __restrict__ v, int ld_v,
                                                                      const float* __restrict__ bd, float* __restrict__ state,
                                                                      const int* __restrict__ seq_start,
                                                                      const int* __restrict__ slots, float* __restrict__ o, int H,
                                                                      int G, int dk, int dv, int vec, int ring_rows) {
  static_assert(DKR % 4 == 0, "a lane keeps whole quads of rows");
  constexpr int DKP = DR_LPC * DKR;             // key width with padding (zeros)
  constexpr int NQ = DKR / 4;                   // quads per lane
  constexpr int ROW = 2 * DKP + 12;             // floats of a ring entry: q | k | 8 values | beta, decay, k.q | 1 unused
  extern __shared__ __align__(16) float ring[];
  int tid = threadIdx.x;
  int j0 = blockIdx.x * 8, h = blockIdx.y, b = blockIdx.z;
  int g = h / (H / G);
  // The block's slice of the state, dk rows of 8 columns (one 32-byte sector a row), goes through shared memory both
  // ways so that every access to the state tensor covers whole sectors, whichever lanes keep which rows.
  float* stage = ring + ring_rows * ROW;        // [dk][9]; ring_rows is DR_RING, or 0 when no sequence of the step needs the ring
  float* Sblock = state + (((size_t)slots[b] * H + h) * dk) * dv + j0;
  for (int i = tid; i < dk * 8; i += DR_THREADS + 32) {
    int d = i >> 3, c = i & 7;
    stage[d * 9 + c] = j0 + c < dv ? Sblock[(size_t)d * dv + c] : 0.f;
  }
  __syncthreads();
  int t0 = seq_start[b], t1 = seq_start[b + 1];
  const bool direct = t1 - t0 <= DR_DIRECT_MAX; // a decode step's one row (or a few): straight from global memory, no ring
  if (!direct && (dk != DKP || j0 + 8 > dv)) {  // padding that no copy touches must read as zero
    for (int i = tid; i < DR_RING * ROW; i += DR_THREADS + 32) ring[i] = 0.f;
    __syncthreads();
  }
  int batches = (t1 - t0 + DR_BATCH - 1) / DR_BATCH;
  // Both kinds of warps pass the same two barriers per batch: (A) the batch before is done with, its half of the
  // ring may be filled again; (B) this batch has landed.
  if (tid >= DR_THREADS) {
    if (direct) return;
    // ---- the copying warp: batches i + 1 .. i + DR_NB - 1 are on their way while batch i is worked on
    int lane = tid - DR_THREADS;
    const int bd_row = 2 * H + G, k_off = G * dk;
    const float* src_q = qk + (size_t)t0 * ld_qk + (size_t)g * dk;
    const float* src_v = v + (size_t)t0 * ld_v + (size_t)h * dv + j0;
    const float* src_bd = bd + (size_t)t0 * bd_row;
    int t_next = t0;
    auto fill_batch = [&](int slot) {
      for (int i = 0; i < DR_BATCH && t_next < t1; i++, t_next++) {
        float* e = ring + (slot * DR_BATCH + i) * ROW;
        if (vec) {
          for (int d = 4 * lane; d < dk; d += 128) {
            cp_async16(e + d, src_q + d);
            cp_async16(e + DKP + d, src_q + k_off + d);
          }
          if (lane < 2 && j0 + 4 * lane < dv) cp_async16(e + 2 * DKP + 4 * lane, src_v + 4 * lane);
        } else {
          for (int d = lane; d < dk; d += 32) {
            cp_async4(e + d, src_q + d);
            cp_async4(e + DKP + d, src_q + k_off + d);
          }
          if (lane < 8 && j0 + lane < dv) cp_async4(e + 2 * DKP + lane, src_v + lane);
        }
        if (lane == 8) cp_async4(e + 2 * DKP + 8, src_bd + h);
        if (lane == 9) cp_async4(e + 2 * DKP + 9, src_bd + H + h);
        if (lane == 10) cp_async4(e + 2 * DKP + 10, src_bd + 2 * H + g);
        src_q += ld_qk;
        src_v += ld_v;
        src_bd += bd_row;
      }
      cp_async_commit();
    };
    for (int i = 0; i < DR_NB - 1; i++) fill_batch(i);          // DR_NB - 1 batches are always on their way
    for (int i = 0; i < batches; i++) {
      __syncthreads();                          // (A)
      cp_async_wait<DR_NB - 2>();               // batch i has landed; the later ones may still be under way
      __syncthreads();                          // (B)
      fill_batch((i + DR_NB - 1) % DR_NB);      // into the slot batch i - 1 used
    }
    cp_async_wait<0>();
    return;
  }
  // ---- the computing warps
  int r = tid & (DR_LPC - 1), col = tid / DR_LPC, j = j0 + col;
  bool live = j < dv;
  float S[DKR];
#pragma unroll
  for (int i = 0; i < DKR; i++) {
    int d = 4 * DR_LPC * (i >> 2) + 4 * r + (i & 3);
    S[i] = d < dk ? stage[d * 9 + col] : 0.f;
  }
  float* dst_o = o + (size_t)t0 * H * dv + (size_t)h * dv + j;
  const int o_step = H * dv;
  if (direct) {
    const int bd_row = 2 * H + G;
    for (int t = t0; t < t1; t++) {
      const float* gq = qk + (size_t)t * ld_qk + (size_t)g * dk;
      const float* gk = gq + (size_t)G * dk;
      const float* gb = bd + (size_t)t * bd_row;
      float de = gb[H + h], be = gb[h], kdotq = gb[2 * H + g];
      float vv = live ? v[(size_t)t * ld_v + (size_t)h * dv + j] : 0.f;
      float4 kk[NQ], qq[NQ];
#pragma unroll
      for (int m = 0; m < NQ; m++) {
        int d = 4 * DR_LPC * m + 4 * r;
        if (vec) {
          kk[m] = d < dk ? *(const float4*)(gk + d) : make_float4(0.f, 0.f, 0.f, 0.f);
          qq[m] = d < dk ? *(const float4*)(gq + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          kk[m] = make_float4(d < dk ? gk[d] : 0.f, d + 1 < dk ? gk[d + 1] : 0.f, d + 2 < dk ? gk[d + 2] : 0.f, d + 3 < dk ? gk[d + 3] : 0.f);
          qq[m] = make_float4(d < dk ? gq[d] : 0.f, d + 1 < dk ? gq[d + 1] : 0.f, d + 2 < dk ? gq[d + 2] : 0.f, d + 3 < dk ? gq[d + 3] : 0.f);
        }
      }
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
      for (int m = 0; m < NQ; m++) {
        a0 += S[4 * m] * kk[m].x; a1 += S[4 * m + 1] * kk[m].y; a2 += S[4 * m + 2] * kk[m].z; a3 += S[4 * m + 3] * kk[m].w;
        c0 += S[4 * m] * qq[m].x; c1 += S[4 * m + 1] * qq[m].y; c2 += S[4 * m + 2] * qq[m].z; c3 += S[4 * m + 3] * qq[m].w;
      }
      float sk = (a0 + a1) + (a2 + a3), sq = (c0 + c1) + (c2 + c3);
#pragma unroll
      for (int w = 1; w < DR_LPC; w <<= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, w);
        sq += __shfl_xor_sync(0xffffffffu, sq, w);
      }
      float u = be * (vv - de * sk);
      float oj = de * sq + u * kdotq;
#pragma unroll
      for (int m = 0; m < NQ; m++) {
        S[4 * m] = de * S[4 * m] + kk[m].x * u; S[4 * m + 1] = de * S[4 * m + 1] + kk[m].y * u;
        S[4 * m + 2] = de * S[4 * m + 2] + kk[m].z * u; S[4 * m + 3] = de * S[4 * m + 3] + kk[m].w * u;
      }
      if (live && r == 0) *dst_o = oj;
      dst_o += o_step;
    }
  }
  for (int ib = 0; ib < (direct ? 0 : batches); ib++) {
    __syncthreads();                            // (A)
    __syncthreads();                            // (B)
    int n = min(DR_BATCH, t1 - t0 - ib * DR_BATCH);
    const float* e = ring + (ib % DR_NB) * DR_BATCH * ROW;
    for (int i = 0; i < n; i++, e += ROW) {
      float de = e[2 * DKP + 9], be = e[2 * DKP + 8], vv = e[2 * DKP + col], kdotq = e[2 * DKP + 10];
      float4 kk[NQ], qq[NQ];
#pragma unroll
      for (int m = 0; m < NQ; m++) {
        kk[m] = *(const float4*)&e[DKP + 4 * DR_LPC * m + 4 * r];
        qq[m] = *(const float4*)&e[4 * DR_LPC * m + 4 * r];
      }
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
      for (int m = 0; m < NQ; m++) {
        a0 += S[4 * m] * kk[m].x; a1 += S[4 * m + 1] * kk[m].y; a2 += S[4 * m + 2] * kk[m].z; a3 += S[4 * m + 3] * kk[m].w;
        c0 += S[4 * m] * qq[m].x; c1 += S[4 * m + 1] * qq[m].y; c2 += S[4 * m + 2] * qq[m].z; c3 += S[4 * m + 3] * qq[m].w;
      }
      float sk = (a0 + a1) + (a2 + a3), sq = (c0 + c1) + (c2 + c3);      // of the old state: S_old^T k and S_old^T q
#pragma unroll
      for (int w = 1; w < DR_LPC; w <<= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, w);
        sq += __shfl_xor_sync(0xffffffffu, sq, w);
      }
      float u = be * (vv - de * sk);
      float oj = de * sq + u * kdotq;
#pragma unroll
      for (int m = 0; m < NQ; m++) {
        S[4 * m] = de * S[4 * m] + kk[m].x * u; S[4 * m + 1] = de * S[4 * m + 1] + kk[m].y * u;
        S[4 * m + 2] = de * S[4 * m + 2] + kk[m].z * u; S[4 * m + 3] = de * S[4 * m + 3] + kk[m].w * u;
      }
      if (live && r == 0) *dst_o = oj;
      dst_o += o_step;
    }
  }
#pragma unroll
  for (int i = 0; i < DKR; i++) {
    int d = 4 * DR_LPC * (i >> 2) + 4 * r + (i & 3);
    if (d < dk) stage[d * 9 + col] = S[i];
  }
  asm volatile("bar.sync 1, %0;" ::"n"(DR_THREADS) : "memory");      // the computing threads only: the copying warp has left
  for (int i = tid; i < dk * 8; i += DR_THREADS) {
    int d = i >> 3, c = i & 7;
    if (j0 + c < dv) Sblock[(size_t)d * dv + c] = stage[d * 9 + c];
  }
}

// Read-out: y[t][h][:] = o / sqrt(mean(o^2) + eps) * w[:] * silu(gate[t][h][:]); a warp per (row, head).
template <typename A>
__global__ void gated_unit_rms_kernel(const float* __restrict__ o, const A* __restrict__ gate, int ld_gate,
                                      const void* __restrict__ w, int w_f32, A* __restrict__ y, int T, int H, int dv, float eps) {
  int lane = threadIdx.x & 31;
  size_t idx = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= (size_t)T * H) return;
  size_t t = idx / H, h = idx % H;
  const float* orow = o + (t * H + h) * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss += orow[j] * orow[j];
  ss = warp_sum(ss);
  float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int j = lane; j < dv; j += 32) {
    float gt = silu_f(to_f32(gate[t * ld_gate + h * dv + j]));
    y[(t * H + h) * dv + j] = from_f32<A>(orow[j] * inv * load_w(w, w_f32, j) * gt);
  }
}

// ------------------------------------------------------------------ real-gated linear recurrence
// Channel c of width W lies in block c / bs of the gates; gates[block][t][0..bs) is the raw recurrence gate,
// [bs..2bs) the raw input gate (block-diagonal products of u, float). r = sigmoid(. + ra_b), i = sigmoid(. + ri_b),
// a = exp(-8 r softplus(lam)); S = a S + sqrt(1 - a^2) i u from the sequence's state [slot][W];
// out[t][c] = S * gelu_tanh(yraw[t][c] + y_b[c]).
struct LruArgs {
  const float* gates; const float* u; const void* yraw; int ld_y;
  const void* ra_b; const void* ri_b; const void* lam; const void* y_b; int w_f32;
  float* state; const int* seq_start; const int* slots; void* out;
  int T, W, bs;
};

struct LruChannel {       // what a thread knows of its channel
  float sp, rb, ib, yb;
  const float* gb;
  int c, cc, bs;
};

__device__ __forceinline__ LruChannel lru_channel(const LruArgs& p, int c) {
  LruChannel ch;
  ch.c = c; ch.bs = p.bs; ch.cc = c % p.bs;
  ch.sp = softplus_f(load_w(p.lam, p.w_f32, c));
  ch.rb = load_w(p.ra_b, p.w_f32, c); ch.ib = load_w(p.ri_b, p.w_f32, c); ch.yb = load_w(p.y_b, p.w_f32, c);
  ch.gb = p.gates + (size_t)(c / p.bs) * p.T * 2 * p.bs;
  return ch;
}

// a_t and b_t of S_t = a_t S_{t-1} + b_t for row t
__device__ __forceinline__ void lru_terms(const LruArgs& p, const LruChannel& ch, int t, float& a, float& bt) {
  float r = sigmoid_f(ch.gb[(size_t)t * 2 * ch.bs + ch.cc] + ch.rb);
  float i = sigmoid_f(ch.gb[(size_t)t * 2 * ch.bs + ch.bs + ch.cc] + ch.ib);
  float log_a = -8.0f * r * ch.sp;
  a = expf(log_a);
  bt = sqrtf(-expm1f(2.0f * log_a)) * (i * p.u[(size_t)t * p.W + ch.c]);      // 1 - a^2 without cancellation
}

// A thread per (sequence, channel) walks the sequence's rows: the decode step, and short portions.
template <typename A>
__global__ void rglru_scan_kernel(LruArgs p) {
  int b = blockIdx.x;
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.W) return;
  LruChannel ch = lru_channel(p, c);
  float* sp_state = p.state + (size_t)p.slots[b] * p.W + c;
  float S = *sp_state;
  int t0 = p.seq_start[b], t1 = p.seq_start[b + 1];
  for (int t = t0; t < t1; t++) {
    float a, bt;
    lru_terms(p, ch, t, a, bt);
    S = a * S + bt;
    ((A*)p.out)[(size_t)t * p.W + c] = from_f32<A>(S * gelu_tanh_f(to_f32(((const A*)p.yraw)[(size_t)t * p.ld_y + c]) + ch.yb));
  }
  *sp_state = S;
}

// Long portions, in three kernels. The rows of a sequence are cut into pieces of LRU_PIECE. (1) A thread per
// (piece, channel) runs its piece from S = 0 and leaves the piece's product of a and its end value:
// S_end = prod * S_start + end. (2) A thread per (sequence, channel) carries the state from piece to piece
// and leaves every piece's S_start (the sequence's state is advanced here). (3) A thread per (piece, channel)
// runs its piece again from S_start and writes the rows. `pieces` = most pieces of any sequence.
#define LRU_PIECE 16
template <typename A>
__global__ void rglru_piece_kernel(LruArgs p, float* __restrict__ prod, float* __restrict__ end, int pieces) {
  int b = blockIdx.x / pieces, k = blockIdx.x % pieces;
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  int t0 = p.seq_start[b] + k * LRU_PIECE, t1 = min(p.seq_start[b + 1], t0 + LRU_PIECE);
  if (c >= p.W || t0 >= t1) return;
  LruChannel ch = lru_channel(p, c);
  float P = 1.f, S = 0.f;
  for (int t = t0; t < t1; t++) {
    float a, bt;
    lru_terms(p, ch, t, a, bt);
    S = a * S + bt;
    P *= a;
  }
  prod[(size_t)blockIdx.x * p.W + c] = P;
  end[(size_t)blockIdx.x * p.W + c] = S;
}

__global__ void rglru_carry_kernel(LruArgs p, const float* __restrict__ prod, float* __restrict__ end, int pieces) {
  int b = blockIdx.x;
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= p.W) return;
  float* sp_state = p.state + (size_t)p.slots[b] * p.W + c;
  float S = *sp_state;
  int n = p.seq_start[b + 1] - p.seq_start[b];
  int used = (n + LRU_PIECE - 1) / LRU_PIECE;
  for (int k0 = 0; k0 < used; k0 += 8) {        // eight pieces' terms fetched together, then chained
    float P[8], E[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      size_t at = ((size_t)b * pieces + min(k0 + i, used - 1)) * p.W + c;
      P[i] = prod[at];
      E[i] = end[at];
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      if (k0 + i < used) {
        end[((size_t)b * pieces + k0 + i) * p.W + c] = S;      // from here on: the piece's start value
        S = P[i] * S + E[i];
      }
    }
  }
  *sp_state = S;
}

template <typename A>
__global__ void rglru_write_kernel(LruArgs p, const float* __restrict__ start, int pieces) {
  int b = blockIdx.x / pieces, k = blockIdx.x % pieces;
  int c = blockIdx.y * blockDim.x + threadIdx.x;
  int t0 = p.seq_start[b] + k * LRU_PIECE, t1 = min(p.seq_start[b + 1], t0 + LRU_PIECE);
  if (c >= p.W || t0 >= t1) return;
  LruChannel ch = lru_channel(p, c);
  float S = start[(size_t)blockIdx.x * p.W + c];
  for (int t = t0; t < t1; t++) {
    float a, bt;
    lru_terms(p, ch, t, a, bt);
    S = a * S + bt;
    ((A*)p.out)[(size_t)t * p.W + c] = from_f32<A>(S * gelu_tanh_f(to_f32(((const A*)p.yraw)[(size_t)t * p.ld_y + c]) + ch.yb));
  }
}
