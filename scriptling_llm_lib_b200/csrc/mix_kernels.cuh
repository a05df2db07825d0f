// Kernels of further mixers and feed-forwards, and of the norm that stands around them:
//   - a norm without statistics (tanh(alpha v) w + b), fused with the residual sum in front of it and with the same
//     kind of norm applied to the addend before it joins the stream;
//   - elementwise activations of a feed-forward's hidden rows;
//   - linear attention with a fixed decay per head (a matrix state per head), worked in pieces of rows;
//   - a read-out norm over the whole row with a gate;
//   - attention over a cached latent: one vector per position that all heads share (store, query absorption,
//     scores and sums over the latent, expansion to value heads);
//   - the selective scan (a state vector per channel whose decay, input and read-out depend on the token);
//   - routed experts: the router, grouping of (token, expert) pairs by expert, and the experts' products.
//
// All of them work on the packed rows of a step (seq_start[b] .. seq_start[b + 1] are the rows of sequence b, in
// order of position) and find a sequence's state through slots[b]. State, sums, scores, norms, gates and decays are
// float32 whatever the element type A of activations and weights.
#pragma once
#include "common.cuh"

namespace mix {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
template <typename A> __device__ __forceinline__ float ld_flag(const void* p, int is_f32, size_t i) {
  return is_f32 ? ((const float*)p)[i] : to_f32(((const A*)p)[i]);
}
template <typename A> __device__ __forceinline__ void st_flag(void* p, int is_f32, size_t i, float v) {
  if (is_f32) ((float*)p)[i] = v;
  else ((A*)p)[i] = from_f32<A>(v);
}

// ------------------------------------------------------------------ residual sum + norm without statistics
// a = sum of the addend's parts (one [T, d] tensor of the element type or float32, or P float32 partial sums);
// with a norm of its own: a <- tanh(pa * a) * pw + pb. v = x[row] + a (x updated in place when rows == nullptr and
// there is an addend). out[r] = tanh(alpha * v) * w + b. Every element on its own: no sums over the row.
struct DytArgs {
  float* x;
  const void* y; int y_f32; int n_parts; long long part_stride;
  const void* pw; const void* pb; float palpha; int has_post; int p_f32;
  const int* rows;
  const void* w; const void* b; float alpha; int w_f32;
  void* out; int out_f32;
  int d;
};

template <typename A> __device__ __forceinline__ float4 ld4_flag(const void* p, int is_f32, size_t i) {
  return is_f32 ? ld4((const float*)p + i) : ld4((const A*)p + i);
}

template <typename A>
__global__ void dyt_add_norm_kernel(DytArgs p, int vec) {
  int r = blockIdx.x;
  size_t in = p.rows ? (size_t)p.rows[r] : (size_t)r;
  bool update = p.rows == nullptr && p.y != nullptr;
  if (vec) {                                      // four elements a thread: d and every buffer's start are multiples of four
    for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * 4; j < p.d; j += gridDim.y * blockDim.x * 4) {
      float4 v = *(const float4*)(p.x + in * p.d + j);
      if (p.y) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < p.n_parts; k++) {
          float4 t = ld4_flag<A>(p.y, p.y_f32, (size_t)k * p.part_stride + in * p.d + j);
          a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
        }
        if (p.has_post) {
          float4 w = *(const float4*)((const float*)p.pw + j), b = *(const float4*)((const float*)p.pb + j);
          a.x = tanhf(p.palpha * a.x) * w.x + b.x; a.y = tanhf(p.palpha * a.y) * w.y + b.y;
          a.z = tanhf(p.palpha * a.z) * w.z + b.z; a.w = tanhf(p.palpha * a.w) * w.w + b.w;
        }
        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
        if (update) *(float4*)(p.x + in * p.d + j) = v;
      }
      if (p.out) {
        float4 w = *(const float4*)((const float*)p.w + j), b = *(const float4*)((const float*)p.b + j);
        float4 y = make_float4(tanhf(p.alpha * v.x) * w.x + b.x, tanhf(p.alpha * v.y) * w.y + b.y, tanhf(p.alpha * v.z) * w.z + b.z,
                               tanhf(p.alpha * v.w) * w.w + b.w);
        if (p.out_f32) st4((float*)p.out + (size_t)r * p.d + j, y);
        else st4((A*)p.out + (size_t)r * p.d + j, y);
      }
    }
    return;
  }
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < p.d; j += gridDim.y * blockDim.x) {
    float v = p.x[in * p.d + j];
    if (p.y) {
      float a = 0.f;
      for (int k = 0; k < p.n_parts; k++) a += ld_flag<A>(p.y, p.y_f32, (size_t)k * p.part_stride + in * p.d + j);
      if (p.has_post) a = tanhf(p.palpha * a) * load_w(p.pw, p.p_f32, j) + load_w(p.pb, p.p_f32, j);
      v += a;
      if (update) p.x[in * p.d + j] = v;
    }
    if (p.out) st_flag<A>(p.out, p.out_f32, (size_t)r * p.d + j, tanhf(p.alpha * v) * load_w(p.w, p.w_f32, j) + load_w(p.b, p.w_f32, j));
  }
}

// ------------------------------------------------------------------ activations in place
// kind 1: the tanh form of gelu; 2: the square of relu; 3: silu
__device__ __forceinline__ float act_f(float z, int kind) {
  return kind == 1 ? gelu_tanh_f(z) : kind == 2 ? (z > 0.f ? z * z : 0.f) : silu_f(z);
}
template <typename A>
__global__ void act_inplace_kernel(A* __restrict__ x, long long n, int kind, int vec) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {                                      // eight elements a thread: n and the buffer's start are multiples of eight
    i *= 8;
    if (i >= n) return;
    F8 v = ld8(x + i);
#pragma unroll
    for (int e = 0; e < 8; e++) v.f[e] = act_f(v.f[e], kind);
    st8(x + i, v);
    return;
  }
  if (i >= n) return;
  x[i] = from_f32<A>(act_f(to_f32(x[i]), kind));
}

// ------------------------------------------------------------------ linear attention with a decay per head
// Per head: S_t = decay * S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, with q, k, v = silu of the projected rows (columns
// q_col, k_col, v_col of `proj`, heads side by side). A block owns VT value columns of one head of one sequence and
// walks the sequence's rows in pieces of at most C rows. Within a piece of n rows (decay^m written g^m):
//   P[i][j] = g^(i-j) q_i . k_j (j <= i);  o_i = g^(i+1) S^T q_i + sum_j P[i][j] v_j;
//   S <- g^n S + sum_j g^(n-1-j) k_j v_j^T.
// All in float32 out of shared memory, 4 x 4 outputs a thread. Warps 0-3 do this work; warps 4-7 fetch the next
// piece's rows meanwhile (SiLU applied) into the other of two buffers. The state [slot][head][D][V] is read at the
// start and written at the end.
__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// A tile [rows][cols_p] of SiLU(src) into shared memory by 128 threads (`lt` among them): src rows `ld` apart, rows
// r >= n and columns c >= cols are zero. All loads of a batch are asked for before the first is used, so that a tile
// costs a few trips to memory and not one per element. vec: eight elements a load (cols a multiple of 8 and equal to
// cols_p, every row's start 16-byte aligned).
template <typename A>
__device__ __forceinline__ void stage_silu_tile(float* __restrict__ dst, int dst_ld, const A* __restrict__ src, int ld, int n,
                                                int rows, int cols, int cols_p, int lt, int vec) {
  if (vec) {
    int chunks = cols_p / 8, total = rows * chunks;
    for (int base = 0; base < total; base += 128 * 4) {
      F8 v[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int i = base + u * 128 + lt;
        int r = i / chunks, c = (i % chunks) * 8;
        if (i < total && r < n) v[u] = ld8(src + (size_t)r * ld + c);
        else {
#pragma unroll
          for (int e = 0; e < 8; e++) v[u].f[e] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int i = base + u * 128 + lt;
        if (i >= total) continue;
        int r = i / chunks, c = (i % chunks) * 8;
        float* d = dst + (size_t)r * dst_ld + c;
        *(float4*)d = make_float4(silu_f(v[u].f[0]), silu_f(v[u].f[1]), silu_f(v[u].f[2]), silu_f(v[u].f[3]));
        *(float4*)(d + 4) = make_float4(silu_f(v[u].f[4]), silu_f(v[u].f[5]), silu_f(v[u].f[6]), silu_f(v[u].f[7]));
      }
    }
    return;
  }
  int total = rows * cols_p;
  for (int base = 0; base < total; base += 128 * 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      int i = base + u * 128 + lt;
      int r = i / cols_p, c = i % cols_p;
      v[u] = (i < total && r < n && c < cols) ? to_f32(src[(size_t)r * ld + c]) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      int i = base + u * 128 + lt;
      if (i < total) dst[(size_t)(i / cols_p) * dst_ld + i % cols_p] = silu_f(v[u]);
    }
  }
}

template <typename A>
__global__ void __launch_bounds__(256) lin_attn_decay_kernel(const A* __restrict__ proj, int ld, int q_col, int k_col, int v_col,
                                                             const float* __restrict__ decay, float* __restrict__ state,
                                                             const int* __restrict__ seq_start, const int* __restrict__ slots,
                                                             float* __restrict__ o, int H, int D, int V, int VT, int C,
                                                             int vec_qk, int vec_v) {
  extern __shared__ __align__(16) float sm[];
  int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * VT;
  int vt = min(VT, V - c0);
  int Dp = (D + 3) & ~3, VTp = (VT + 3) & ~3;
  int qs_ld = Dp + 4;
  size_t qk_size = (size_t)C * qs_ld, v_size = (size_t)C * VTp;
  float* S = sm;                                  // [Dp][VTp]
  float* qs0 = S + (size_t)Dp * VTp;              // two buffers of [C][qs_ld] queries, [C][qs_ld] keys, [C][VTp] values
  float* P = qs0 + 2 * (2 * qk_size + v_size);    // [C][C]
  float* pw = P + (size_t)C * C;                  // [C + 2] powers of the decay
  int tid = threadIdx.x;
  bool loader = tid >= 128;
  int ct = tid & 127;                             // index among the computing (or the fetching) threads
  float g = decay[h];
  if (tid == 0) {
    float a = 1.f;
    for (int i = 0; i <= C + 1; i++) { pw[i] = a; a *= g; }
  }
  float* st = state + ((size_t)slots[b] * H + h) * D * V;
  int r_begin = seq_start[b], r_end = seq_start[b + 1];
  int n_pieces = (r_end - r_begin + C - 1) / C;

  auto stage = [&](int piece) {
    float* qs = qs0 + (size_t)(piece & 1) * (2 * qk_size + v_size);
    float* ks = qs + qk_size;
    float* vs = ks + qk_size;
    int r0 = r_begin + piece * C;
    int n = min(C, r_end - r0);
    const A* base = proj + (size_t)r0 * ld;
    stage_silu_tile<A>(qs, qs_ld, base + q_col + (size_t)h * D, ld, n, C, D, Dp, ct, vec_qk);
    stage_silu_tile<A>(ks, qs_ld, base + k_col + (size_t)h * D, ld, n, C, D, Dp, ct, vec_qk);
    stage_silu_tile<A>(vs, VTp, base + v_col + (size_t)h * V + c0, ld, n, C, vt, VTp, ct, vec_v && vt == VTp);
  };

  if (loader) {
    if (n_pieces > 0) stage(0);
  } else {
    for (int i = ct; i < Dp * VTp; i += 128) {
      int d = i / VTp, c = i % VTp;
      S[i] = (d < D && c < vt) ? st[(size_t)d * V + c0 + c] : 0.f;
    }
  }
  __syncthreads();
  for (int piece = 0; piece < n_pieces; piece++) {
    if (loader) {
      if (piece + 1 < n_pieces) stage(piece + 1);
      __syncthreads();
      continue;
    }
    const float* qs = qs0 + (size_t)(piece & 1) * (2 * qk_size + v_size);
    const float* ks = qs + qk_size;
    const float* vs = ks + qk_size;
    int r0 = r_begin + piece * C;
    int n = min(C, r_end - r0);
    // scores inside the piece: 2 x 2 a thread (C is even), blocks above the diagonal are left at zero
    int c2 = C / 2;
    for (int it = ct; it < c2 * c2; it += 128) {
      int qi = (it / c2) * 2, kj = (it % c2) * 2;
      float s00 = 0.f, s01 = 0.f, s10 = 0.f, s11 = 0.f;
      if (kj <= qi + 1 && qi < n) {
        const float4* a0 = (const float4*)(qs + qi * qs_ld);
        const float4* a1 = (const float4*)(qs + (qi + 1) * qs_ld);
        const float4* b0 = (const float4*)(ks + kj * qs_ld);
        const float4* b1 = (const float4*)(ks + (kj + 1) * qs_ld);
        for (int d = 0; d < Dp / 4; d++) {
          float4 x0 = a0[d], x1 = a1[d], y0 = b0[d], y1 = b1[d];
          s00 += (x0.x * y0.x + x0.y * y0.y) + (x0.z * y0.z + x0.w * y0.w);
          s01 += (x0.x * y1.x + x0.y * y1.y) + (x0.z * y1.z + x0.w * y1.w);
          s10 += (x1.x * y0.x + x1.y * y0.y) + (x1.z * y0.z + x1.w * y0.w);
          s11 += (x1.x * y1.x + x1.y * y1.y) + (x1.z * y1.z + x1.w * y1.w);
        }
        s00 = kj <= qi ? s00 * pw[qi - kj] : 0.f;
        s01 = kj + 1 <= qi ? s01 * pw[qi - kj - 1] : 0.f;
        s10 = s10 * pw[min(qi + 1 - kj, C)];
        s11 = kj <= qi ? s11 * pw[qi - kj] : 0.f;
        if (qi + 1 >= n) { s10 = 0.f; s11 = 0.f; }
      }
      P[qi * C + kj] = s00; P[qi * C + kj + 1] = s01;
      P[(qi + 1) * C + kj] = s10; P[(qi + 1) * C + kj + 1] = s11;
    }
    bar_compute();
    // outputs of the piece: RT rows x 4 columns a thread, RT = 4 where that gives every thread work, else 1
    int c4 = VTp / 4;
    if (((n + 3) / 4) * c4 >= 128) {
      int n4 = (n + 3) / 4;
      for (int it = ct; it < n4 * c4; it += 128) {
        int i0 = (it / c4) * 4, cc = (it % c4) * 4;
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
          for (int c = 0; c < 4; c++) acc[a][c] = 0.f;
        for (int d = 0; d < D; d++) {
          float4 sv = *(const float4*)(S + (size_t)d * VTp + cc);
#pragma unroll
          for (int a = 0; a < 4; a++) {
            float qv = (i0 + a < C) ? qs[(i0 + a) * qs_ld + d] : 0.f;
            acc[a][0] += qv * sv.x; acc[a][1] += qv * sv.y; acc[a][2] += qv * sv.z; acc[a][3] += qv * sv.w;
          }
        }
#pragma unroll
        for (int a = 0; a < 4; a++) {
          float f = pw[min(i0 + a + 1, C + 1)];
#pragma unroll
          for (int c = 0; c < 4; c++) acc[a][c] *= f;
        }
        int jmax = min(i0 + 3, n - 1);
        for (int j = 0; j <= jmax; j++) {
          float4 vv = *(const float4*)(vs + (size_t)j * VTp + cc);
#pragma unroll
          for (int a = 0; a < 4; a++) {
            float pv = (i0 + a < C) ? P[(i0 + a) * C + j] : 0.f;      // zero above the diagonal
            acc[a][0] += pv * vv.x; acc[a][1] += pv * vv.y; acc[a][2] += pv * vv.z; acc[a][3] += pv * vv.w;
          }
        }
#pragma unroll
        for (int a = 0; a < 4; a++) {
          if (i0 + a >= n) continue;
          float* orow = o + (size_t)(r0 + i0 + a) * H * V + (size_t)h * V + c0 + cc;
#pragma unroll
          for (int c = 0; c < 4; c++)
            if (cc + c < vt) orow[c] = acc[a][c];
        }
      }
    } else {
      for (int it = ct; it < n * c4; it += 128) {
        int i = it / c4, cc = (it % c4) * 4;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        const float* qrow = qs + i * qs_ld;
        for (int d = 0; d < D; d++) {
          float4 sv = *(const float4*)(S + (size_t)d * VTp + cc);
          float qv = qrow[d];
          a0 += qv * sv.x; a1 += qv * sv.y; a2 += qv * sv.z; a3 += qv * sv.w;
        }
        float f = pw[i + 1];
        a0 *= f; a1 *= f; a2 *= f; a3 *= f;
        for (int j = 0; j <= i; j++) {
          float4 vv = *(const float4*)(vs + (size_t)j * VTp + cc);
          float pv = P[i * C + j];
          a0 += pv * vv.x; a1 += pv * vv.y; a2 += pv * vv.z; a3 += pv * vv.w;
        }
        float* orow = o + (size_t)(r0 + i) * H * V + (size_t)h * V + c0 + cc;
        if (cc < vt) orow[0] = a0;
        if (cc + 1 < vt) orow[1] = a1;
        if (cc + 2 < vt) orow[2] = a2;
        if (cc + 3 < vt) orow[3] = a3;
      }
    }
    bar_compute();
    // the state after the piece: 4 key dims x 4 columns a thread
    float gn = pw[n];
    int d4 = Dp / 4;
    for (int it = ct; it < d4 * c4; it += 128) {
      int d0 = (it / c4) * 4, cc = (it % c4) * 4;
      float acc[4][4];
#pragma unroll
      for (int a = 0; a < 4; a++) {
        float4 sv = *(const float4*)(S + (size_t)(d0 + a) * VTp + cc);
        acc[a][0] = gn * sv.x; acc[a][1] = gn * sv.y; acc[a][2] = gn * sv.z; acc[a][3] = gn * sv.w;
      }
      for (int j = 0; j < n; j++) {
        float f = pw[n - 1 - j];
        float4 kv = *(const float4*)(ks + (size_t)j * qs_ld + d0);
        float4 vv = *(const float4*)(vs + (size_t)j * VTp + cc);
        vv.x *= f; vv.y *= f; vv.z *= f; vv.w *= f;
        acc[0][0] += kv.x * vv.x; acc[0][1] += kv.x * vv.y; acc[0][2] += kv.x * vv.z; acc[0][3] += kv.x * vv.w;
        acc[1][0] += kv.y * vv.x; acc[1][1] += kv.y * vv.y; acc[1][2] += kv.y * vv.z; acc[1][3] += kv.y * vv.w;
        acc[2][0] += kv.z * vv.x; acc[2][1] += kv.z * vv.y; acc[2][2] += kv.z * vv.z; acc[2][3] += kv.z * vv.w;
        acc[3][0] += kv.w * vv.x; acc[3][1] += kv.w * vv.y; acc[3][2] += kv.w * vv.z; acc[3][3] += kv.w * vv.w;
      }
#pragma unroll
      for (int a = 0; a < 4; a++)
        *(float4*)(S + (size_t)(d0 + a) * VTp + cc) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    }
    __syncthreads();
  }
  if (!loader)
    for (int i = ct; i < Dp * VTp; i += 128) {
      int d = i / VTp, c = i % VTp;
      if (d < D && c < vt) st[(size_t)d * V + c0 + c] = S[i];
    }
}

// ------------------------------------------------------------------ read-out norm over the whole row with a gate
// y[t] = o[t] / sqrt(mean(o[t]^2) + eps) * w * gate(g[t]); gate_act 1: sigmoid, 2: silu. o float32 [T, W]; g a column
// slice of the projections (element type).
template <typename A>
__global__ void gated_row_rms_kernel(const float* __restrict__ o, const A* __restrict__ g, int ldg, const void* __restrict__ w,
                                     int w_f32, A* __restrict__ y, int W, float eps, int gate_act) {
  __shared__ float red[32];
  int t = blockIdx.x;
  const float* orow = o + (size_t)t * W;
  float ss = 0.f;
  for (int j = threadIdx.x; j < W; j += blockDim.x) ss += orow[j] * orow[j];
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int j = threadIdx.x; j < W; j += blockDim.x) {
    float z = to_f32(g[(size_t)t * ldg + j]);
    float gate = gate_act == 1 ? sigmoid_f(z) : silu_f(z);
    y[(size_t)t * W + j] = from_f32<A>(orow[j] * inv * load_w(w, w_f32, j) * gate);
  }
}

// ------------------------------------------------------------------ attention over a cached latent
// A position keeps one vector [R + P]: the latent c (the first R of the down-projection's output divided by their
// root mean square, times a weight) and a key part of P dims rotated by its position, shared by all heads. Pages:
// [page][SLLM_PAGE][R + P] of the element type.
//
// store: one block per row. Writes [c | rotated key part] at the row's place (when pages != nullptr) and rotates
// the last P dims of every query head in place (the leading `rot` of them, in adjacent pairs, by the table
// [position][rot / 2] of (cos, sin)).
template <typename A>
__global__ void latent_store_kernel(A* __restrict__ q, int ldq, int H, int D, const A* __restrict__ dkv, int ldk,
                                    const void* __restrict__ nw, int nw_f32, float eps, const float2* __restrict__ cos_sin,
                                    int rot, int half, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                    const int* __restrict__ block_table, int max_pages, A* __restrict__ pages, int R, int P) {
  __shared__ float red[32];
  int t = blockIdx.x;
  int pos = tok_pos[t];
  const int hr = rot / 2;
  const float2* cs = cos_sin + (size_t)pos * hr;
  // pair pr of the rotated part: dims (2 pr, 2 pr + 1), or with `half` dims (pr, pr + rot / 2)
  for (int i = threadIdx.x; i < H * hr; i += blockDim.x) {
    int h = i / hr, pr = i % hr;
    A* qp = q + (size_t)t * ldq + (size_t)h * (D + P) + D;
    int a = half ? pr : 2 * pr, b = half ? pr + hr : 2 * pr + 1;
    float u = to_f32(qp[a]), v = to_f32(qp[b]);
    float2 c = cs[pr];
    qp[a] = from_f32<A>(u * c.x - v * c.y);
    qp[b] = from_f32<A>(v * c.x + u * c.y);
  }
  if (!pages) return;
  const A* row = dkv + (size_t)t * ldk;
  float ss = 0.f;
  for (int j = threadIdx.x; j < R; j += blockDim.x) {
    float v = to_f32(row[j]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)R + eps);
  int page = block_table[(size_t)tok_seq[t] * max_pages + pos / SLLM_PAGE];
  A* dst = pages + ((size_t)page * SLLM_PAGE + pos % SLLM_PAGE) * (R + P);
  for (int j = threadIdx.x; j < R; j += blockDim.x) dst[j] = from_f32<A>(to_f32(row[j]) * inv * load_w(nw, nw_f32, j));
  for (int pr = threadIdx.x; pr < hr; pr += blockDim.x) {
    int a = R + (half ? pr : 2 * pr), b = R + (half ? pr + hr : 2 * pr + 1);
    float u = to_f32(row[a]), v = to_f32(row[b]);
    float2 c = cs[pr];
    dst[a] = from_f32<A>(u * c.x - v * c.y);
    dst[b] = from_f32<A>(v * c.x + u * c.y);
  }
  for (int j = 2 * hr + threadIdx.x; j < P; j += blockDim.x) dst[R + j] = row[R + j];
}

// gather: the cached vectors of a step's rows side by side, dense[t] = pages[place of (sequence, position) of row t].
template <typename A>
__global__ void latent_gather_kernel(const A* __restrict__ pages, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                     const int* __restrict__ block_table, int max_pages, A* __restrict__ dense, int W) {
  int t = blockIdx.x;
  int pos = tok_pos[t];
  const A* src = pages + ((size_t)block_table[(size_t)tok_seq[t] * max_pages + pos / SLLM_PAGE] * SLLM_PAGE + pos % SLLM_PAGE) * W;
  for (int j = threadIdx.x; j < W; j += blockDim.x) dense[(size_t)t * W + j] = src[j];
}

// heads: keys and values per head for a prompt that starts at position 0, laid out as pages of their own so that an
// attention kernel for keys and values of one width `hd` >= max(D + P, V) can run on them. kv[t] = [Wuk c | Wuv c] (H D
// and H V wide), dense[t][R ..] the rotated key part. kt[page][h][place] = [key of head h | rotated part | 0 ..],
// vt[...] = [value of head h | 0 ..], qt[t][h] = [query of head h (D + P) | 0 ..]; the page of (sequence, position) comes
// from `table` [sequences][max_pages].
template <typename A>
__global__ void latent_heads_kernel(const A* __restrict__ q, int ldq, const A* __restrict__ kv, int ldkv,
                                    const A* __restrict__ dense, int ldd, int R, const int* __restrict__ tok_pos,
                                    const int* __restrict__ tok_seq, const int* __restrict__ table, int max_pages,
                                    A* __restrict__ kt, A* __restrict__ vt, A* __restrict__ qt, int H, int D, int P, int V, int hd) {
  int t = blockIdx.x, h = blockIdx.y;
  int pos = tok_pos[t];
  size_t at = (((size_t)table[(size_t)tok_seq[t] * max_pages + pos / SLLM_PAGE] * H + h) * SLLM_PAGE + pos % SLLM_PAGE) * hd;
  const A zero = from_f32<A>(0.f);
  for (int j = threadIdx.x; j < hd; j += blockDim.x) {
    kt[at + j] = j < D ? kv[(size_t)t * ldkv + (size_t)h * D + j] : (j < D + P ? dense[(size_t)t * ldd + R + j - D] : zero);
    vt[at + j] = j < V ? kv[(size_t)t * ldkv + (size_t)H * D + (size_t)h * V + j] : zero;
    qt[((size_t)t * H + h) * hd + j] = j < D + P ? q[(size_t)t * ldq + (size_t)h * (D + P) + j] : zero;
  }
}

// absorb: the query a head asks the latent with. qa[t][h] = scale * [ Wuk_h^T q_unrot | q_rot ] (float32, R + P
// wide), Wuk_h = rows h D .. h D + D - 1 of the stored [H D, R] matrix. A block takes up to 8 rows of one head;
// threads run over the latent's columns, so a row of the matrix is read in one piece.
#define MIX_ABSORB_ROWS 8
template <typename A>
__global__ void __launch_bounds__(128) latent_absorb_kernel(const A* __restrict__ q, int ldq, const A* __restrict__ wuk,
                                                            float* __restrict__ qa, int T, int H, int D, int P, int R,
                                                            float scale) {
  extern __shared__ __align__(16) float sm[];     // [8][D]
  int h = blockIdx.y, t0 = blockIdx.x * MIX_ABSORB_ROWS;
  int n = min(MIX_ABSORB_ROWS, T - t0);
  for (int i = threadIdx.x; i < MIX_ABSORB_ROWS * D; i += blockDim.x) {
    int r = i / D, d = i % D;
    sm[i] = r < n ? to_f32(q[(size_t)(t0 + r) * ldq + (size_t)h * (D + P) + d]) * scale : 0.f;
  }
  __syncthreads();
  const A* w = wuk + (size_t)h * D * R;
  int c = blockIdx.z * blockDim.x + threadIdx.x;  // a latent column a thread
  if (c < R) {
    float acc[MIX_ABSORB_ROWS];
#pragma unroll
    for (int r = 0; r < MIX_ABSORB_ROWS; r++) acc[r] = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; d++) {
      float wv = to_f32(w[(size_t)d * R + c]);
#pragma unroll
      for (int r = 0; r < MIX_ABSORB_ROWS; r++) acc[r] += sm[r * D + d] * wv;
    }
    for (int r = 0; r < n; r++) qa[((size_t)(t0 + r) * H + h) * (R + P) + c] = acc[r];
  }
  if (blockIdx.z == 0)
    for (int i = threadIdx.x; i < n * P; i += blockDim.x) {
      int r = i / P, j = i % P;
      qa[((size_t)(t0 + r) * H + h) * (R + P) + R + j] = to_f32(q[(size_t)(t0 + r) * ldq + (size_t)h * (D + P) + D + j]) * scale;
    }
}

// scores and sums: one block per (row, group of up to 8 heads, split of the keys), a warp per head. Keys arrive in
// tiles of 32 rows, staged in shared memory as floats once for all heads of the block; a lane scores one key of the
// tile, softmax statistics are renewed once per tile, and the sum over the latent runs with the columns spread over
// the lanes (NV columns a lane). Causal: keys 0 .. pos of the row's sequence. Each split leaves (max, sum, sums over
// the latent) in `part` [T][H][n_split][R + 2]; the expansion merges them.
template <typename A, int NV>
__global__ void __launch_bounds__(256) latent_attn_kernel(const float* __restrict__ qa, const A* __restrict__ pages,
                                                          const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                                          const int* __restrict__ block_table, int max_pages,
                                                          float* __restrict__ part, int H, int R, int P, int n_split, int vec) {
  extern __shared__ __align__(16) float sm[];
  int W = R + P, Wp = W + 1;
  int t = blockIdx.x, h0 = blockIdx.y * 8, sp = blockIdx.z;
  int nh = min(8, H - h0);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int nthreads = blockDim.x;
  float* qs = sm;                                 // [8][W]
  float* Ks = qs + 8 * W;                         // [32][Wp]
  int pos = tok_pos[t];
  const int* pt = block_table + (size_t)tok_seq[t] * max_pages;
  for (int i = threadIdx.x; i < nh * W; i += nthreads) qs[i] = qa[((size_t)t * H + h0) * W + i];
  int n_tiles = pos / 32 + 1;
  int per = (n_tiles + n_split - 1) / n_split;
  int tile_lo = sp * per, tile_hi = min(n_tiles, tile_lo + per);
  float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) acc[i] = 0.f;
  bool active = wid < nh;
  const float* myq = qs + wid * W;
  for (int tile = tile_lo; tile < tile_hi; tile++) {
    int k0 = tile * 32;
    int nk = min(32, pos + 1 - k0);
    __syncthreads();
    // a tile of 32 keys lies inside one page (32 divides the page size): one look-up for the tile, then whole rows a warp
    const A* tile_src = pages + ((size_t)pt[k0 / SLLM_PAGE] * SLLM_PAGE + k0 % SLLM_PAGE) * W;
    constexpr int VEC = 16 / sizeof(A);
    if (vec) {
      int chunks = W / VEC, total = 32 * chunks;
      for (int base = 0; base < total; base += 4 * nthreads) {       // four loads a thread in flight
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          int i = base + u * nthreads + threadIdx.x;
          int kr = i / chunks, d = (i % chunks) * VEC;
          raw[u] = (i < total && kr < nk) ? *(const uint4*)(tile_src + (size_t)kr * W + d) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          int i = base + u * nthreads + threadIdx.x;
          if (i >= total) continue;
          int kr = i / chunks, d = (i % chunks) * VEC;
          float* dst = Ks + kr * Wp + d;
          if constexpr (sizeof(A) == 2) {
            const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw[u];
#pragma unroll
            for (int e = 0; e < 4; e++) { dst[2 * e] = __low2float(h2[e]); dst[2 * e + 1] = __high2float(h2[e]); }
          } else {
            dst[0] = __uint_as_float(raw[u].x); dst[1] = __uint_as_float(raw[u].y);
            dst[2] = __uint_as_float(raw[u].z); dst[3] = __uint_as_float(raw[u].w);
          }
        }
      }
    } else {
      for (int i = threadIdx.x; i < 32 * W; i += nthreads) {
        int kr = i / W, d = i % W;
        Ks[kr * Wp + d] = kr < nk ? to_f32(tile_src[(size_t)kr * W + d]) : 0.f;
      }
    }
    __syncthreads();
    if (!active) continue;
    float sc = -INFINITY;
    if (lane < nk) {
      const float* kr = Ks + lane * Wp;
      float s0 = 0.f, s1 = 0.f;
      int d = 0;
      for (; d + 1 < W; d += 2) { s0 += myq[d] * kr[d]; s1 += myq[d + 1] * kr[d + 1]; }
      if (d < W) s0 += myq[d] * kr[d];
      sc = s0 + s1;
    }
    float m_new = fmaxf(m, warp_max(sc));
    float c = expf(m - m_new);
    float pwt = lane < nk ? expf(sc - m_new) : 0.f;
    l = l * c + warp_sum(pwt);
    m = m_new;
#pragma unroll
    for (int i = 0; i < NV; i++) acc[i] *= c;
    for (int j = 0; j < nk; j++) {
      float pj = __shfl_sync(0xffffffffu, pwt, j);
      const float* kr = Ks + j * Wp;
#pragma unroll
      for (int i = 0; i < NV; i++) {
        int col = lane + 32 * i;
        if (col < R) acc[i] += pj * kr[col];
      }
    }
  }
  if (!active) return;
  float* dst = part + (((size_t)t * H + h0 + wid) * n_split + sp) * (R + 2);
  if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
  for (int i = 0; i < NV; i++) {
    int col = lane + 32 * i;
    if (col < R) dst[2 + col] = acc[i];
  }
}

// The same with 16-byte accesses to shared memory, for widths that are multiples of four (R and R + P): the tile's row
// stride is a multiple of four floats and an odd number of 16-byte groups (lanes that read different rows hit different
// banks), a lane scores its key four dims a load, and in the sum over the latent it owns groups of four neighbouring
// columns (4 lane + 128 i). Four times fewer loads from shared memory per multiply-add than the kernel above.
template <typename A, int NV4>
__global__ void __launch_bounds__(256) latent_attn_vec_kernel(const float* __restrict__ qa, const A* __restrict__ pages,
                                                              const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                                              const int* __restrict__ block_table, int max_pages,
                                                              float* __restrict__ part, int H, int R, int P, int n_split, int Wp) {
  extern __shared__ __align__(16) float sm[];
  int W = R + P;
  int t = blockIdx.x, h0 = blockIdx.y * 8, sp = blockIdx.z;
  int nh = min(8, H - h0);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int nthreads = blockDim.x;
  float* qs = sm;                                 // [8][W]
  float* Ks = qs + 8 * W;                         // [32][Wp]
  int pos = tok_pos[t];
  const int* pt = block_table + (size_t)tok_seq[t] * max_pages;
  for (int i = threadIdx.x; i < nh * W; i += nthreads) qs[i] = qa[((size_t)t * H + h0) * W + i];
  int n_tiles = pos / 32 + 1;
  int per = (n_tiles + n_split - 1) / n_split;
  int tile_lo = sp * per, tile_hi = min(n_tiles, tile_lo + per);
  float m = -INFINITY, l = 0.f, acc[NV4][4];
#pragma unroll
  for (int i = 0; i < NV4; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  bool active = wid < nh;
  const float4* myq = (const float4*)(qs + wid * W);
  constexpr int VEC = 16 / sizeof(A);
  for (int tile = tile_lo; tile < tile_hi; tile++) {
    int k0 = tile * 32;
    int nk = min(32, pos + 1 - k0);
    __syncthreads();
    const A* tile_src = pages + ((size_t)pt[k0 / SLLM_PAGE] * SLLM_PAGE + k0 % SLLM_PAGE) * W;
    int chunks = W / VEC, total = 32 * chunks;
    for (int base = 0; base < total; base += 4 * nthreads) {         // four loads a thread in flight
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int i = base + u * nthreads + threadIdx.x;
        int kr = i / chunks, d = (i % chunks) * VEC;
        raw[u] = (i < total && kr < nk) ? *(const uint4*)(tile_src + (size_t)kr * W + d) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int i = base + u * nthreads + threadIdx.x;
        if (i >= total) continue;
        int kr = i / chunks, d = (i % chunks) * VEC;
        float* dst = Ks + kr * Wp + d;
        if constexpr (sizeof(A) == 2) {
          const __nv_bfloat162* h2 = (const __nv_bfloat162*)&raw[u];
          *(float4*)dst = make_float4(__low2float(h2[0]), __high2float(h2[0]), __low2float(h2[1]), __high2float(h2[1]));
          *(float4*)(dst + 4) = make_float4(__low2float(h2[2]), __high2float(h2[2]), __low2float(h2[3]), __high2float(h2[3]));
        } else {
          *(float4*)dst = make_float4(__uint_as_float(raw[u].x), __uint_as_float(raw[u].y), __uint_as_float(raw[u].z),
                                      __uint_as_float(raw[u].w));
        }
      }
    }
    __syncthreads();
    if (!active) continue;
    float sc = -INFINITY;
    if (lane < nk) {
      const float4* kr = (const float4*)(Ks + lane * Wp);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
      for (int d = 0; d < W / 4; d++) {
        float4 x = myq[d], y = kr[d];
        s0 += x.x * y.x + x.y * y.y;
        s1 += x.z * y.z + x.w * y.w;
      }
      sc = s0 + s1;
    }
    float m_new = fmaxf(m, warp_max(sc));
    float c = expf(m - m_new);
    float pwt = lane < nk ? expf(sc - m_new) : 0.f;
    l = l * c + warp_sum(pwt);
    m = m_new;
#pragma unroll
    for (int i = 0; i < NV4; i++) { acc[i][0] *= c; acc[i][1] *= c; acc[i][2] *= c; acc[i][3] *= c; }
    for (int j = 0; j < nk; j++) {
      float pj = __shfl_sync(0xffffffffu, pwt, j);
      const float* kr = Ks + j * Wp;
#pragma unroll
      for (int i = 0; i < NV4; i++) {
        int col = 4 * lane + 128 * i;
        if (col < R) {
          float4 y = *(const float4*)(kr + col);
          acc[i][0] += pj * y.x; acc[i][1] += pj * y.y; acc[i][2] += pj * y.z; acc[i][3] += pj * y.w;
        }
      }
    }
  }
  if (!active) return;
  float* dst = part + (((size_t)t * H + h0 + wid) * n_split + sp) * (R + 2);
  if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
  for (int i = 0; i < NV4; i++) {
    int col = 4 * lane + 128 * i;
    if (col < R) { dst[2 + col] = acc[i][0]; dst[3 + col] = acc[i][1]; dst[4 + col] = acc[i][2]; dst[5 + col] = acc[i][3]; }
  }
}

// merge: olat[t][h] = sum_s w_s acc_s / sum_s w_s l_s, w_s = exp(m_s - max m): the splits' sums over the latent as one
// normalised vector [R] per (row, head). The first warp weighs the splits once (a lane takes splits lane, lane + 32, ...),
// then every thread adds its columns over the splits with loads that do not depend on one another.
#define MIX_MERGE_SPLITS 64
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ part, float* __restrict__ olat, int R, int n_split) {
  __shared__ float w[MIX_MERGE_SPLITS];
  __shared__ float s_inv;
  size_t item = blockIdx.x;                       // t * H + h
  const float* p0 = part + item * n_split * (R + 2);
  if (n_split <= MIX_MERGE_SPLITS) {
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      float ms[MIX_MERGE_SPLITS / 32], ls[MIX_MERGE_SPLITS / 32], mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < MIX_MERGE_SPLITS / 32; i++) {
        int s2 = lane + 32 * i;
        ms[i] = s2 < n_split ? p0[(size_t)s2 * (R + 2)] : -INFINITY;
        ls[i] = s2 < n_split ? p0[(size_t)s2 * (R + 2) + 1] : 0.f;
        mx = fmaxf(mx, ms[i]);
      }
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float den = 0.f;
#pragma unroll
      for (int i = 0; i < MIX_MERGE_SPLITS / 32; i++) {
        float ws = ms[i] > -INFINITY ? expf(ms[i] - mx) : 0.f;
        w[lane + 32 * i] = ws;
        den += ws * ls[i];
      }
      for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
      if (lane == 0) s_inv = 1.0f / den;
    }
    __syncthreads();
    const float inv = s_inv;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
      float a = 0.f;
#pragma unroll 8
      for (int s = 0; s < n_split; s++) {
        const float ws = w[s];                    // a split without keys left its sums unwritten: they are not read
        if (ws != 0.f) a += ws * p0[(size_t)s * (R + 2) + 2 + c];
      }
      olat[item * R + c] = a * inv;
    }
    return;
  }
  float mx = -INFINITY;
  for (int s = 0; s < n_split; s++) mx = fmaxf(mx, p0[(size_t)s * (R + 2)]);
  float den = 0.f;
  for (int s = 0; s < n_split; s++) {
    float ms = p0[(size_t)s * (R + 2)];
    if (ms > -INFINITY) den += expf(ms - mx) * p0[(size_t)s * (R + 2) + 1];
  }
  float inv = 1.0f / den;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_split; s++) {
      float ms = p0[(size_t)s * (R + 2)];
      if (ms > -INFINITY) a += expf(ms - mx) * p0[(size_t)s * (R + 2) + 2 + c];
    }
    olat[item * R + c] = a * inv;
  }
}

// expand: maps the summed latents to the head's values: out[t][h V + v] = Wuv[h V + v] . olat[t][h]. A block takes up
// to 8 rows of one head and four output columns, a warp a column.
template <typename A>
__global__ void __launch_bounds__(128) latent_expand_kernel(const float* __restrict__ olat, const A* __restrict__ wuv,
                                                            A* __restrict__ out, int ldo, int T, int H, int V, int R) {
  extern __shared__ __align__(16) float sm[];     // [8][R]
  int h = blockIdx.y, t0 = blockIdx.x * MIX_ABSORB_ROWS;
  int n = min(MIX_ABSORB_ROWS, T - t0);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < MIX_ABSORB_ROWS * R; i += blockDim.x) {
    int r = i / R, c = i % R;
    sm[i] = r < n ? olat[((size_t)(t0 + r) * H + h) * R + c] : 0.f;
  }
  __syncthreads();
  int v = blockIdx.z * 4 + wid;
  if (v >= V) return;
  const A* w = wuv + ((size_t)h * V + v) * R;
  float acc[MIX_ABSORB_ROWS];
#pragma unroll
  for (int r = 0; r < MIX_ABSORB_ROWS; r++) acc[r] = 0.f;
#pragma unroll 4
  for (int c = lane; c < R; c += 32) {
    float wv = to_f32(w[c]);
#pragma unroll
    for (int r = 0; r < MIX_ABSORB_ROWS; r++) acc[r] += sm[r * R + c] * wv;
  }
#pragma unroll
  for (int r = 0; r < MIX_ABSORB_ROWS; r++) acc[r] = warp_sum(acc[r]);
  if (lane == 0)
    for (int r = 0; r < n; r++) out[(size_t)(t0 + r) * ldo + (size_t)h * V + v] = from_f32<A>(acc[r]);
}

// ------------------------------------------------------------------ the selective scan
// Per channel c a state S[c][0..N): for each row dt = softplus(dt_raw[c] + dt_bias[c]);
// S[c][n] <- exp(dt * A[c][n]) * S[c][n] + dt * x[c] * B[n];  y[c] = sum_n S[c][n] * C[n] + D[c] * x[c];  out = y * silu(z[c]),
// A = -exp(A_log). 4, 8 or 16 lanes share a channel (state n = lane + L i: the more states, the more lanes, so that a row
// costs a lane few dependent steps and the GPU gets warps enough); a block takes 128 / L channels of one sequence and
// walks its rows, which a second set of warps stages in shared memory ahead of the walk. x, z, B, C: column slices of
// buffers of the element type; dt_raw float32.
struct ScanArgs {
  const void* x; int ldx;
  const float* dt_raw; int lddt;
  const void* dt_bias; const void* a_log; const void* dskip; int w_f32;
  const void* bc; int ldbc; int b_col; int c_col;
  const void* z; int ldz;
  float* state;
  const int* seq_start; const int* slots;
  void* out; int ldo;
  int I, N;
};

template <typename A, int NPL, int L, int MIX_SCAN_ROWS>      // MIX_SCAN_ROWS: rows staged at a time
__global__ void __launch_bounds__(256) selective_scan_kernel(ScanArgs p) {
  // Warps 0-3 walk the rows: L lanes share a channel (state n = lane + L i), 128 / L channels a block. Warps 4-7 stage the
  // next MIX_SCAN_ROWS rows meanwhile: step sizes with their softplus, inputs, gates with their SiLU (the block's channels
  // a row) and the rows' B and C (N each), two buffers in turn.
  extern __shared__ __align__(16) float sm[];
  constexpr int CPB = 128 / L;                    // channels a block
  const int N = p.N, per_buf = MIX_SCAN_ROWS * (3 * CPB + 2 * N);
  int b = blockIdx.y, ch0 = blockIdx.x * CPB;
  int r_begin = p.seq_start[b], r_end = p.seq_start[b + 1];
  int n_chunks = (r_end - r_begin + MIX_SCAN_ROWS - 1) / MIX_SCAN_ROWS;
  const A* xs = (const A*)p.x;
  const A* zs = (const A*)p.z;
  const A* bcs = (const A*)p.bc;
  A* out = (A*)p.out;
  bool loader = threadIdx.x >= 128;
  int lt = threadIdx.x - 128;

  auto stage = [&](int chunk) {
    float* buf = sm + (size_t)(chunk & 1) * per_buf;
    float *dt_s = buf, *x_s = buf + MIX_SCAN_ROWS * CPB, *z_s = x_s + MIX_SCAN_ROWS * CPB, *b_s = z_s + MIX_SCAN_ROWS * CPB,
          *c_s = b_s + MIX_SCAN_ROWS * N;
    int r0 = r_begin + chunk * MIX_SCAN_ROWS;
    int n = min(MIX_SCAN_ROWS, r_end - r0);
    // all loads of the chunk first, the arithmetic behind them
    constexpr int PER = (MIX_SCAN_ROWS * CPB + 127) / 128;
    float dtr[PER], xr[PER], zr[PER];
#pragma unroll
    for (int u = 0; u < PER; u++) {
      int i = lt + 128 * u;
      int r = i / CPB, ch = ch0 + i % CPB;
      bool ok = i < MIX_SCAN_ROWS * CPB && r < n && ch < p.I;
      dtr[u] = ok ? p.dt_raw[(size_t)(r0 + r) * p.lddt + ch] + load_w(p.dt_bias, p.w_f32, ch) : 0.f;
      xr[u] = ok ? to_f32(xs[(size_t)(r0 + r) * p.ldx + ch]) : 0.f;
      zr[u] = ok ? to_f32(zs[(size_t)(r0 + r) * p.ldz + ch]) : 0.f;
    }
    for (int base = 0; base < MIX_SCAN_ROWS * N; base += 128 * 8) {
      float bv[8], cv[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        int i = base + lt + 128 * u;
        int r = i / N, nn = i % N;
        bool ok = i < MIX_SCAN_ROWS * N && r < n;
        const A* row = bcs + (size_t)(r0 + r) * p.ldbc;
        bv[u] = ok ? to_f32(row[p.b_col + nn]) : 0.f;
        cv[u] = ok ? to_f32(row[p.c_col + nn]) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        int i = base + lt + 128 * u;
        if (i < MIX_SCAN_ROWS * N) { b_s[i] = bv[u]; c_s[i] = cv[u]; }
      }
    }
#pragma unroll
    for (int u = 0; u < PER; u++) {
      int i = lt + 128 * u;
      if (i >= MIX_SCAN_ROWS * CPB) continue;
      int r = i / CPB, ch = ch0 + i % CPB;
      bool ok = r < n && ch < p.I;
      dt_s[i] = ok ? softplus_f(dtr[u]) : 0.f;
      x_s[i] = xr[u];
      z_s[i] = ok ? silu_f(zr[u]) : 0.f;
    }
  };

  int cc = (threadIdx.x & 127) / L, l = threadIdx.x % L;
  int ch = ch0 + cc;
  bool live = !loader && ch < p.I;
  int c = min(ch, p.I - 1);
  float Areg[NPL], S[NPL];
  float* st = p.state + ((size_t)p.slots[b] * p.I + c) * N;
  float dsk = 0.f;
  if (!loader) {
#pragma unroll
    for (int i = 0; i < NPL; i++) {
      int n = l + L * i;
      Areg[i] = n < N ? -expf(load_w(p.a_log, p.w_f32, (size_t)c * N + n)) : 0.f;
      S[i] = n < N ? st[n] : 0.f;
    }
    dsk = load_w(p.dskip, p.w_f32, c);
  } else if (n_chunks > 0) {
    stage(0);
  }
  __syncthreads();
  for (int chunk = 0; chunk < n_chunks; chunk++) {
    if (loader) {
      if (chunk + 1 < n_chunks) stage(chunk + 1);
    } else {
      const float* buf = sm + (size_t)(chunk & 1) * per_buf;
      const float *dt_s = buf, *x_s = buf + MIX_SCAN_ROWS * CPB, *z_s = x_s + MIX_SCAN_ROWS * CPB, *b_s = z_s + MIX_SCAN_ROWS * CPB,
                  *c_s = b_s + MIX_SCAN_ROWS * N;
      int r0 = r_begin + chunk * MIX_SCAN_ROWS;
      int n = min(MIX_SCAN_ROWS, r_end - r0);
#pragma unroll 4
      for (int r = 0; r < n; r++) {
        float dt = dt_s[r * CPB + cc], xv = x_s[r * CPB + cc];
        float dx = dt * xv;
        const float* brow = b_s + r * N;
        const float* crow = c_s + r * N;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; i++) {
          int nn = l + L * i;
          if (nn < N) {
            S[i] = expf(dt * Areg[i]) * S[i] + dx * brow[nn];
            acc += S[i] * crow[nn];
          }
        }
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (l == 0 && live) out[(size_t)(r0 + r) * p.ldo + ch] = from_f32<A>((acc + dsk * xv) * z_s[r * CPB + cc]);
      }
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPL; i++) {
      int n = l + L * i;
      if (n < N) st[n] = S[i];
    }
  }
}

// ------------------------------------------------------------------ routed experts
// router: a warp per token. z [T][E] float32 are the router's logits (a product of the library, float32 sums).
// mode 2: s = softmax(z + bias) over all experts; runs of experts as in mode 0 but a run is rated by its best s alone; the
// `top` open experts with the highest s are picked and count with s * scale as it is (not renormalised).
// mode 1: c = z + bias (corr; may be null), the `top` experts with the highest c are picked and count with the
// softmax over the picked c alone (n_groups 1, scale unused). mode 0:
// s = sigmoid(z), c = s + correction. The experts are cut into n_groups runs of equal length, a run is rated by its best
// two c added up, the `keep` best-rated runs stay open, and among the open experts the `top` with the highest c are picked
// (ties: the lower index). Expert e then counts with s_e / (sum of the picked s + 1e-20) * scale.
// idx int32 [T][top], wgt float32 [T][top].
#define MIX_ROUTE_WARPS 4
__global__ void __launch_bounds__(32 * MIX_ROUTE_WARPS) moe_route_kernel(const float* __restrict__ z, const void* __restrict__ corr,
                                                                         int corr_f32, int* __restrict__ idx,
                                                                         float* __restrict__ wgt, int T, int E, int n_groups,
                                                                         int keep, int top, float scale, int mode) {
  extern __shared__ __align__(16) float sm[];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int t = blockIdx.x * MIX_ROUTE_WARPS + wid;
  if (t >= T) return;
  float* s = sm + (size_t)wid * (2 * E + n_groups);   // [E] sigmoid scores
  float* ch = s + E;                                  // [E] the picking scores c (-inf once picked or in a run that is shut)
  float* gs = ch + E;                                 // [n_groups]
  for (int e = lane; e < E; e += 32) {
    float zz = z[(size_t)t * E + e];
    float sg = mode ? zz + (corr ? load_w(corr, corr_f32, e) : 0.f) : sigmoid_f(zz);
    s[e] = sg;
    ch[e] = mode ? sg : sg + load_w(corr, corr_f32, e);
  }
  __syncwarp();
  if (mode == 2) {          // the scores are the softmax of z + bias over ALL experts; they rate and weigh
    float mx = -INFINITY, sum = 0.f;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    for (int e = lane; e < E; e += 32) {
      float ex = expf(s[e] - mx);
      s[e] = ex;
      sum += ex;
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
      s[e] *= inv;
      ch[e] = s[e];
    }
    __syncwarp();
  }
  int gsz = E / n_groups;
  if (n_groups > 1) {
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b2 = -INFINITY;
      for (int j = 0; j < gsz; j++) {
        float v = ch[g * gsz + j];
        if (v > a) { b2 = a; a = v; }
        else if (v > b2) b2 = v;
      }
      gs[g] = (gsz > 1 && mode != 2) ? a + b2 : a;       // mode 2 rates a run by its best member alone
    }
    __syncwarp();
    // the groups that are not kept: n_groups - keep rounds of taking the smallest out (ties: the higher index goes)
    for (int round = 0; round < n_groups - keep; round++) {
      float best = INFINITY;
      int bi = -1;
      for (int g = lane; g < n_groups; g += 32) {
        float v = gs[g];
        if (v <= best && v < INFINITY) { best = v; bi = g; }      // later (higher) index wins ties inside a lane
      }
      for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ob < best || (ob == best && oi > bi))) { best = ob; bi = oi; }
      }
      if (bi < 0) break;
      if (lane == 0) gs[bi] = INFINITY;           // marks a group that is shut out
      for (int j = lane; j < gsz; j += 32) ch[bi * gsz + j] = -INFINITY;
      __syncwarp();
    }
  }
  __syncwarp();
  float sum = 0.f, first = 0.f;
  for (int k = 0; k < top; k++) {
    float best = -INFINITY;
    int bi = -1;
    for (int e = lane; e < E; e += 32) {
      float v = ch[e];
      if (v > best) { best = v; bi = e; }         // the lower index wins ties inside a lane
    }
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi >= 0 && (bi < 0 || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
    }
    if (bi < 0) bi = 0;                           // fewer experts allowed than asked for: cannot happen with a checked configuration
    if (k == 0) first = s[bi];                    // the largest picked logit: the softmax's reference (mode 1)
    float sv = mode == 1 ? expf(s[bi] - first) : s[bi];
    sum += sv;
    if (lane == 0) {
      idx[(size_t)t * top + k] = bi;
      wgt[(size_t)t * top + k] = sv;
      ch[bi] = -INFINITY;
    }
    __syncwarp();
  }
  float f = mode == 2 ? scale : mode ? 1.0f / sum : scale / (sum + 1e-20f);
  for (int k = lane; k < top; k += 32) wgt[(size_t)t * top + k] *= f;
}

// The clamped gate of an expert: g' * sigmoid(alpha * g') * (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit).
// limit <= 0 stands for the gate without a clamp: silu(g) * u.
__device__ __forceinline__ float glu_clamp_f(float g, float u, float limit, float alpha) {
  if (!(limit > 0.f)) return g * sigmoid_f(g) * u;       // no limit: the plain gate silu(g) * u
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoid_f(alpha * g) * (u + 1.0f);
}
// Where gate f and up f of an expert lie among its 2 F stacked rows (and among the 2 F sums of a row): F gate rows and
// then F up rows, or `tiled` (F a multiple of 8): tiles of 16 rows, 8 gate rows and then their 8 up rows, which is the
// order the tensor-core product's gated store wants.
__device__ __forceinline__ int glu_gate_at(int f, int F, int tiled) { return tiled ? ((f >> 3) << 4) + (f & 7) : f; }
__device__ __forceinline__ int glu_up_at(int f, int F, int tiled) { return tiled ? ((f >> 3) << 4) + 8 + (f & 7) : F + f; }
// gu [rows][2 F]: the gate and up sums of a row; out[row][f] = the clamped gate of its pair f.
// Rows from *rows_used on (when given) are left alone.
template <typename A>
__global__ void glu_clamp_kernel(const A* __restrict__ gu, A* __restrict__ out, int rows, int F, float limit, float alpha,
                                 const int* __restrict__ rows_used, int tiled) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * F) return;
  int r = (int)(i / F), f = (int)(i % F);
  if (rows_used && r >= *rows_used) return;
  const A* g = gu + (size_t)r * 2 * F;
  out[i] = from_f32<A>(glu_clamp_f(to_f32(g[glu_gate_at(f, F, tiled)]), to_f32(g[glu_up_at(f, F, tiled)]), limit, alpha));
}

// Few rows (a decode step): every (token, chosen expert) pair on its own, a warp per output column.
//   up:   hid[p][f] = relu(Wup[e_p][f] . h[t_p])^2           p = t * top + k
//         gated (Wup holds F gate rows and F up rows per expert; 1: one run after the other, 2: in tiles of 16):
//         hid[p][f] = glu(gate row f . h, up row f . h)
//   down: out[k][t][j] = wgt[p] * (Wdown[e_p][j] . hid[p])    float32 partial sums over k, added by the reader
template <typename A>
__device__ __forceinline__ float warp_dot(const A* __restrict__ x, const A* __restrict__ w, int K, int lane, int vec) {
  float a0 = 0.f, a1 = 0.f;
  if (vec) {                                      // eight elements a lane and pass: K and both rows' starts are multiples of 8 elements
#pragma unroll 2
    for (int k = lane * 8; k < K; k += 256) {
      F8 xv = ld8(x + k), wv = ld8(w + k);
      a0 += xv.f[0] * wv.f[0] + xv.f[2] * wv.f[2] + xv.f[4] * wv.f[4] + xv.f[6] * wv.f[6];
      a1 += xv.f[1] * wv.f[1] + xv.f[3] * wv.f[3] + xv.f[5] * wv.f[5] + xv.f[7] * wv.f[7];
    }
  } else {
    for (int k = lane; k < K; k += 32) a0 += to_f32(x[k]) * to_f32(w[k]);
  }
  return warp_sum(a0 + a1);
}

template <typename A>
__global__ void __launch_bounds__(128) moe_pair_up_kernel(const A* __restrict__ h, int ldh, const A* __restrict__ wup,
                                                          const int* __restrict__ idx, A* __restrict__ hid, int top, int K, int F,
                                                          int vec, int gated, float limit, float alpha) {
  int p = blockIdx.y;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int f = blockIdx.x * nw + wid;
  if (f >= F) return;
  const A* x = h + (size_t)(p / top) * ldh;
  if (gated) {
    const A* we = wup + (size_t)idx[p] * 2 * F * K;
    float g = warp_dot(x, we + (size_t)glu_gate_at(f, F, gated == 2) * K, K, lane, vec);
    float u = warp_dot(x, we + (size_t)glu_up_at(f, F, gated == 2) * K, K, lane, vec);
    if (lane == 0) hid[(size_t)p * F + f] = from_f32<A>(glu_clamp_f(g, u, limit, alpha));
    return;
  }
  float a = warp_dot(x, wup + ((size_t)idx[p] * F + f) * K, K, lane, vec);
  if (lane == 0) hid[(size_t)p * F + f] = from_f32<A>(a > 0.f ? a * a : 0.f);
}

template <typename A>
__global__ void __launch_bounds__(128) moe_pair_down_kernel(const A* __restrict__ hid, const A* __restrict__ wdown,
                                                            const int* __restrict__ idx, const float* __restrict__ wgt,
                                                            float* __restrict__ out, int T, int top, int F, int N, int vec) {
  int p = blockIdx.y;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int j = blockIdx.x * nw + wid;
  if (j >= N) return;
  float a = warp_dot(hid + (size_t)p * F, wdown + ((size_t)idx[p] * N + j) * F, F, lane, vec);
  if (lane == 0) out[((size_t)(p % top) * T + p / top) * N + j] = wgt[p] * a;
}

// Many rows (a prompt step): the pairs are grouped by expert. count: how many pairs every expert got;
// offsets: their prefix sums (one block); place: every pair's row in the grouped order (pairs of one expert in
// any order: a row's result does not depend on its place).
__global__ void moe_count_kernel(const int* __restrict__ idx, int n_pairs, int* __restrict__ counts) {
  int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p < n_pairs) atomicAdd(&counts[idx[p]], 1);
}
// offsets[e]: the first grouped row of expert e, every expert's range rounded up to a multiple of `pad` rows (1: none;
// offsets[E]: the end). With tile_group: tile_group[t] = the expert whose range holds rows t * pad .. (the last expert
// with rows for the tiles behind all ranges: they hold no pair).
__global__ void moe_offsets_kernel(int* __restrict__ counts, int* __restrict__ offsets, int E, int pad,
                                   int* __restrict__ tile_group, int n_tiles) {
  extern __shared__ int cnt[];                    // the counts fetched by all threads at once; one thread then adds them up
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    cnt[e] = counts[e];
    counts[e] = 0;                                // reused as the fill counters of the placing pass
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, t = 0;
    for (int e = 0; e < E; e++) {
      offsets[e] = a;
      a += (cnt[e] + pad - 1) / pad * pad;
      if (tile_group)
        for (; t < n_tiles && t * pad < a; t++) tile_group[t] = e;
    }
    offsets[E] = a;
    if (tile_group)
      for (; t < n_tiles; t++) tile_group[t] = E - 1;
  }
}
__global__ void moe_place_kernel(const int* __restrict__ idx, int n_pairs, const int* __restrict__ offsets,
                                 int* __restrict__ fill, int* __restrict__ pair_of_row, int* __restrict__ row_of_pair) {
  int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs) return;
  int e = idx[p];
  int row = offsets[e] + atomicAdd(&fill[e], 1);
  pair_of_row[row] = p;
  if (row_of_pair) row_of_pair[p] = row;
}

// The grouped rows' inputs side by side: xs[row] = h[pair_of_row[row] / top], zeros for a row that holds no pair.
template <typename A>
__global__ void moe_gather_rows_kernel(const A* __restrict__ h, int ldh, const int* __restrict__ pair_of_row, int top,
                                       A* __restrict__ xs, int K, int vec) {
  int row = blockIdx.x;
  int p = pair_of_row[row];
  A* dst = xs + (size_t)row * K;
  if (vec) {                                      // 16 bytes a thread: K * sizeof(A), ldh * sizeof(A) and both starts are multiples
    constexpr int PER = 16 / sizeof(A);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int j = threadIdx.x * PER; j < K; j += blockDim.x * PER)
      *(uint4*)(dst + j) = p >= 0 ? *(const uint4*)(h + (size_t)(p / top) * ldh + j) : zero;
    return;
  }
  for (int j = threadIdx.x; j < K; j += blockDim.x) dst[j] = p >= 0 ? h[(size_t)(p / top) * ldh + j] : from_f32<A>(0.f);
}

// out[t] = sum_k wgt[t][k] * ys[row_of_pair[t * top + k]], the choices in their order: float32 [T, N].
__global__ void moe_combine_kernel(const float* __restrict__ ys, const int* __restrict__ row_of_pair,
                                   const float* __restrict__ wgt, float* __restrict__ out, int top, int N) {
  int t = blockIdx.x;
  for (int j = threadIdx.x; j < N; j += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; k++) a += wgt[(size_t)t * top + k] * ys[(size_t)row_of_pair[(size_t)t * top + k] * N + j];
    out[(size_t)t * N + j] = a;
  }
}

// the same, four columns a thread (N a multiple of four); the choices are added in the same order
__global__ void moe_combine_vec_kernel(const float* __restrict__ ys, const int* __restrict__ row_of_pair,
                                       const float* __restrict__ wgt, float* __restrict__ out, int top, int N) {
  int t = blockIdx.x;
  for (int j = threadIdx.x * 4; j < N; j += blockDim.x * 4) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top; k++) {
      float w = wgt[(size_t)t * top + k];
      float4 v = *(const float4*)(ys + (size_t)row_of_pair[(size_t)t * top + k] * N + j);
      a.x += w * v.x; a.y += w * v.y; a.z += w * v.z; a.w += w * v.w;
    }
    *(float4*)(out + (size_t)t * N + j) = a;
  }
}

// The experts' products over the grouped rows: tiles of 64 rows x 64 columns of one expert, 16 of K at a time
// through shared memory, 4 x 4 outputs a thread, float32 sums. Tile `blockIdx.x` of the rows: the experts' row
// ranges are cut into tiles of 64 in order; a block beyond the last tile leaves.
//   mode 0 (up):   a row's input is h[pair / top]; out: hid[row][col] = relu(acc)^2 (element type)
//   mode 2 (up):   the same input; out: hid[row][col] = acc (element type), for an activation that pairs columns
//   mode 1 (down): a row's input is hid[row]; out[pair % top][pair / top][col] = wgt[pair] * acc (float32)
template <typename A>
__global__ void __launch_bounds__(256) moe_grouped_gemm_kernel(const A* __restrict__ in, int ldin, const A* __restrict__ w,
                                                               const int* __restrict__ offsets, const int* __restrict__ pair_of_row,
                                                               const float* __restrict__ wgt, void* __restrict__ out, int E,
                                                               int top, int T, int K, int N, int mode) {
  __shared__ __align__(16) float As[16][64 + 4];
  __shared__ __align__(16) float Bs[16][64 + 4];
  __shared__ int src_row[64];
  __shared__ int tile_info[3];
  if (threadIdx.x == 0) {
    int want = blockIdx.x, e = 0, found = -1, r0 = 0, r1 = 0;
    for (; e < E; e++) {
      int lo = offsets[e], hi = offsets[e + 1];
      int nt = (hi - lo + 63) / 64;
      if (want < nt) { found = e; r0 = lo + want * 64; r1 = min(hi, r0 + 64); break; }
      want -= nt;
    }
    tile_info[0] = found; tile_info[1] = r0; tile_info[2] = r1;
  }
  __syncthreads();
  int e = tile_info[0], r0 = tile_info[1], r1 = tile_info[2];
  if (e < 0) return;
  int n_rows = r1 - r0;
  int col0 = blockIdx.y * 64;
  if (threadIdx.x < 64) {
    int r = threadIdx.x;
    src_row[r] = r < n_rows ? (mode != 1 ? pair_of_row[r0 + r] / top : r0 + r) : -1;
  }
  __syncthreads();
  const A* wexp = w + (size_t)e * N * K;
  int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;           // columns tx * 4 .., rows ty * 4 ..
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; a++)
#pragma unroll
    for (int c = 0; c < 4; c++) acc[a][c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int r = i >> 4, kk = i & 15;
      int sr = src_row[r];
      float av = (sr >= 0 && k0 + kk < K) ? to_f32(in[(size_t)sr * ldin + k0 + kk]) : 0.f;
      As[kk][r] = av;
      int cidx = col0 + r;
      float bv = (cidx < N && k0 + kk < K) ? to_f32(wexp[(size_t)cidx * K + k0 + kk]) : 0.f;
      Bs[kk][r] = bv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; kk++) {
      float4 av = *(const float4*)&As[kk][ty * 4];
      float4 bv = *(const float4*)&Bs[kk][tx * 4];
      float a4[4] = {av.x, av.y, av.z, av.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int a = 0; a < 4; a++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[a][c] += a4[a] * b4[c];
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; a++) {
    int r = ty * 4 + a;
    if (r >= n_rows) continue;
    if (mode != 1) {
      A* orow = (A*)out + (size_t)(r0 + r) * N;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        int col = col0 + tx * 4 + c;
        if (col < N) orow[col] = from_f32<A>(mode == 2 ? acc[a][c] : acc[a][c] > 0.f ? acc[a][c] * acc[a][c] : 0.f);
      }
    } else {
      int pr = pair_of_row[r0 + r];
      float wv = wgt[pr];
      float* orow = (float*)out + ((size_t)(pr % top) * T + pr / top) * N;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        int col = col0 + tx * 4 + c;
        if (col < N) orow[col] = wv * acc[a][c];
      }
    }
  }
}

}  // namespace mix
