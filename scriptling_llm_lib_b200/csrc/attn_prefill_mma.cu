// Causal attention of a prompt step over the paged cache for key and value widths the tcgen05 kernels do not take
// (keys KD wide, values VD wide, each a multiple of 16 out of a short list; storage rows may be wider). bfloat16 operands on
// mma.sync.m16n8k16 with float accumulation, scores, cap, softmax statistics and sink in float; the weights enter the
// product with the values rounded to bfloat16, as in the library's other tensor-core attention kernels.
//
// One block of four warps: 64 consecutive queries of one sequence and one query head (a warp has 16 of them) against tiles
// of 64 keys (a page). A tile's keys and values come into shared memory with 16-byte cp.async copies, two tiles in turn, so
// the next page is on its way while this one is multiplied. S = Q K^T: the query fragments stay in registers for the whole
// block (read once from global memory), the key fragments are 32-bit reads of the row-major tile (rows padded by 8 elements:
// no bank conflicts). The accumulators of S are the A operand of P V as they stand (two neighbouring 8-key blocks make one
// 16-key step); the value fragments come through ldmatrix with .trans from the row-major tile.
#include "common.cuh"

#define PM_BQ 64
#define PM_BK 64          // = SLLM_PAGE
#define PM_LOG2E 1.4426950408889634f

struct PmArgs {
  const bf16* q;        // [T, q_ld]; head h at columns h * q_hw, its first KD columns used
  int q_ld, q_hw;
  bf16* out;            // [T, out_ld]; head h at columns h * o_hw: VD columns written, the rest of the head's o_hw set to 0
  int out_ld, o_hw;
  const int* seq_start; // [B + 1]
  const int* seq_pos0;  // [B]
  const int* block_table;
  int max_pages;
  const bf16* kpages;   // [pages][G][64][k_w]
  const bf16* vpages;   // [pages][G][64][v_w]
  int k_w, v_w;
  int H, G, window;
  float scale, softcap;
  const float* sink;    // [H] or null
};

__device__ __forceinline__ void pm_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pm_cp16(void* dst, const void* src) {
  uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t pm_pack(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *(uint32_t*)&h;
}

template <int KD, int VD>
__global__ void __launch_bounds__(128) attn_prefill_mma_kernel(PmArgs p) {
  constexpr int KS = KD + 8, VS = VD + 8;          // padded rows of the tiles in shared memory (elements)
  constexpr int KT = PM_BK * KS, VT = PM_BK * VS;  // elements of a key tile and of a value tile
  extern __shared__ __align__(16) bf16 pm_sm[];    // two stages of [key tile | value tile]
  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int row0 = p.seq_start[b], S = p.seq_start[b + 1] - row0;
  const int r0 = qt * PM_BQ;
  if (r0 >= S) return;
  const int nq = min(PM_BQ, S - r0);
  const int pos0 = p.seq_pos0[b];
  const int g_kv = h / (p.H / p.G);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int* bt = p.block_table + (size_t)b * p.max_pages;

  // the warp's 16 queries as A fragments: rows g and g + 8, sixteen dims a step
  uint32_t qa[KD / 16][4];
  {
    const int ra = r0 + warp * 16 + g, rb = ra + 8;
    const bf16* qa_row = p.q + (size_t)(row0 + ra) * p.q_ld + (size_t)h * p.q_hw;
    const bf16* qb_row = p.q + (size_t)(row0 + rb) * p.q_ld + (size_t)h * p.q_hw;
#pragma unroll
    for (int kk = 0; kk < KD / 16; kk++) {
      const int c = kk * 16 + 2 * t;
      qa[kk][0] = ra < S ? *(const uint32_t*)(qa_row + c) : 0u;
      qa[kk][1] = rb < S ? *(const uint32_t*)(qb_row + c) : 0u;
      qa[kk][2] = ra < S ? *(const uint32_t*)(qa_row + c + 8) : 0u;
      qa[kk][3] = rb < S ? *(const uint32_t*)(qb_row + c + 8) : 0u;
    }
  }
  const int k_hi = pos0 + r0 + nq;                                   // one past the last key any query of the block sees
  const int t_lo = first_seen(pos0 + r0, p.window) / PM_BK, t_hi = (k_hi - 1) / PM_BK;

  auto load_tile = [&](int stage, int tile) {
    bf16* ks = pm_sm + (size_t)stage * (KT + VT);
    bf16* vs = ks + KT;
    const int page = bt[tile];
    const size_t base = ((size_t)max(page, 0) * p.G + g_kv) * SLLM_PAGE;
    const bf16* kp = p.kpages + base * p.k_w;
    const bf16* vp = p.vpages + base * p.v_w;
    for (int e = tid; e < PM_BK * (KD / 8); e += 128) {
      const int kk = e / (KD / 8), c = (e % (KD / 8)) * 8;
      if (page >= 0 && tile * PM_BK + kk < k_hi) pm_cp16(ks + kk * KS + c, kp + (size_t)kk * p.k_w + c);
      else *(uint4*)(ks + kk * KS + c) = make_uint4(0, 0, 0, 0);
    }
    for (int e = tid; e < PM_BK * (VD / 8); e += 128) {
      const int kk = e / (VD / 8), c = (e % (VD / 8)) * 8;
      // rows past the last key hold whatever the page held before: their weights are 0, but 0 * NaN is NaN
      if (page >= 0 && tile * PM_BK + kk < k_hi) pm_cp16(vs + kk * VS + c, vp + (size_t)kk * p.v_w + c);
      else *(uint4*)(vs + kk * VS + c) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float o[VD / 8][4];
#pragma unroll
  for (int i = 0; i < VD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;       // rows g and g + 8: running maximum (base 2) and this lane's share of the sum
  const int qpos0 = pos0 + r0 + warp * 16 + g, qpos1 = qpos0 + 8;
  const int first0 = first_seen(qpos0, p.window), first1 = first_seen(qpos1, p.window);
  const float sc = p.softcap > 0.f ? p.scale / p.softcap : p.scale * PM_LOG2E;
  const float cap_l2 = p.softcap * PM_LOG2E;

  load_tile(0, t_lo);
  for (int tile = t_lo; tile <= t_hi; tile++) {
    const int stage = (tile - t_lo) & 1;
    if (tile < t_hi) {
      load_tile(stage ^ 1, tile + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* ks = pm_sm + (size_t)stage * (KT + VT);
    const bf16* vs = ks + KT;
    const int kt = tile * PM_BK;
    // a warp skips the tiles that lie wholly behind its last query (every warp walks the loop: the barriers are the block's)
    if (kt <= pos0 + r0 + warp * 16 + 15 && r0 + warp * 16 < S) {
      float s[8][4];
#pragma unroll
      for (int nb = 0; nb < 8; nb++) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KD / 16; kk++) {
#pragma unroll
        for (int nb = 0; nb < 8; nb++) {
          const bf16* kr = ks + (nb * 8 + g) * KS + kk * 16 + 2 * t;
          pm_mma(s[nb], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], *(const uint32_t*)kr, *(const uint32_t*)(kr + 8));
        }
      }
      // scale (and cap), mask, row maxima over the quad that shares a row
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < 8; nb++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const int key = kt + nb * 8 + 2 * t + (c & 1);
          const int qpos = c < 2 ? qpos0 : qpos1, first = c < 2 ? first0 : first1;
          float v = s[nb][c] * sc;
          if (p.softcap > 0.f) v = cap_l2 * tanhf(v);
          v = (key <= qpos && key >= first) ? v : -INFINITY;
          s[nb][c] = v;
          if (c < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float c0 = n0 == -INFINITY ? 1.f : exp2f(m0 - n0), c1 = n1 == -INFINITY ? 1.f : exp2f(m1 - n1);
      m0 = n0; m1 = n1;
      l0 *= c0; l1 *= c1;
#pragma unroll
      for (int i = 0; i < VD / 8; i++) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
      const float u0 = m0 == -INFINITY ? 0.f : m0, u1 = m1 == -INFINITY ? 0.f : m1;
#pragma unroll
      for (int nb = 0; nb < 8; nb++) {
        s[nb][0] = exp2f(s[nb][0] - u0); s[nb][1] = exp2f(s[nb][1] - u0);
        s[nb][2] = exp2f(s[nb][2] - u1); s[nb][3] = exp2f(s[nb][3] - u1);
        l0 += s[nb][0] + s[nb][1];
        l1 += s[nb][2] + s[nb][3];
      }
      // O += P V, sixteen keys a step; the value fragments of two 8-dim blocks per ldmatrix
#pragma unroll
      for (int kb = 0; kb < 4; kb++) {
        const uint32_t a0 = pm_pack(s[2 * kb][0], s[2 * kb][1]), a1 = pm_pack(s[2 * kb][2], s[2 * kb][3]);
        const uint32_t a2 = pm_pack(s[2 * kb + 1][0], s[2 * kb + 1][1]), a3 = pm_pack(s[2 * kb + 1][2], s[2 * kb + 1][3]);
        const bf16* vrow = vs + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + (lane >> 4) * 8;
#pragma unroll
        for (int nb2 = 0; nb2 < VD / 8; nb2 += 2) {
          uint32_t b0, b1, b2, b3;
          const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vrow + nb2 * 8);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
          pm_mma(o[nb2], a0, a1, a2, a3, b0, b1);
          pm_mma(o[nb2 + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();                     // the stage is free for the tile after the next
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (p.sink != nullptr) {
    const float sk = p.sink[h] * PM_LOG2E;
    l0 = m0 == -INFINITY ? 1.f : l0 + exp2f(sk - m0);
    l1 = m1 == -INFINITY ? 1.f : l1 + exp2f(sk - m1);
  }
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int ra = r0 + warp * 16 + g, rb = ra + 8;
  bf16* oa = p.out + (size_t)(row0 + ra) * p.out_ld + (size_t)h * p.o_hw;
  bf16* ob = p.out + (size_t)(row0 + rb) * p.out_ld + (size_t)h * p.o_hw;
#pragma unroll
  for (int i = 0; i < VD / 8; i++) {
    if (ra < S) *(uint32_t*)(oa + i * 8 + 2 * t) = pm_pack(o[i][0] * i0, o[i][1] * i0);
    if (rb < S) *(uint32_t*)(ob + i * 8 + 2 * t) = pm_pack(o[i][2] * i1, o[i][3] * i1);
  }
  for (int c = VD + 2 * t; c < p.o_hw; c += 8) {       // the head's columns past the values (a padded layout): zeros
    if (ra < S) *(uint32_t*)(oa + c) = 0u;
    if (rb < S) *(uint32_t*)(ob + c) = 0u;
  }
}

template <int KD, int VD>
static int pm_launch(const PmArgs& a, int B, int max_new, cudaStream_t stream) {
  size_t smem = (size_t)2 * PM_BK * ((KD + 8) + (VD + 8)) * sizeof(bf16);
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<KD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  dim3 grid((max_new + PM_BQ - 1) / PM_BQ, a.H, B);
  attn_prefill_mma_kernel<KD, VD><<<grid, 128, smem, stream>>>(a);
  SLLM_RETURN_LAST();
}

// The key widths and value widths the kernel is built for; a caller pads its rows with zeros up to the next one.
SLLM_EXPORT int sllm_attn_prefill_mma_takes(int kd, int vd) {
  return (kd == 64 || kd == 96 || kd == 128 || kd == 192 || kd == 256) && (vd == 64 || vd == 128);
}

// q [T, q_ld] with head h at columns h * q_hw; out [T, out_ld] with head h at columns h * o_hw; kpages [pages][G][64][k_w],
// vpages [pages][G][64][v_w]; kd <= q_hw, k_w and vd <= v_w, o_hw are the widths used. All widths multiples of 8 elements and
// all pointers 16-byte aligned (the copies are 16 bytes wide).
SLLM_EXPORT int sllm_attn_prefill_mma_bf16(const void* q, int q_ld, int q_hw, void* out, int out_ld, int o_hw, const int* seq_start,
                                           const int* seq_pos0, const int* block_table, int max_pages, const void* kpages, int k_w,
                                           const void* vpages, int v_w, int B, int max_new, int H, int G, int kd, int vd, int window,
                                           float scale, float softcap, const float* sink, cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (!sllm_attn_prefill_mma_takes(kd, vd) || G < 1 || H % G != 0 || kd > q_hw || kd > k_w || vd > v_w || vd > o_hw ||
      ((q_ld | q_hw | out_ld | o_hw | k_w | v_w) & 7) || (((uintptr_t)q | (uintptr_t)out | (uintptr_t)kpages | (uintptr_t)vpages) & 15))
    return SLLM_ERR_ARG;
  PmArgs a{(const bf16*)q, q_ld, q_hw, (bf16*)out, out_ld, o_hw, seq_start, seq_pos0, block_table, max_pages, (const bf16*)kpages,
           (const bf16*)vpages, k_w, v_w, H, G, window, scale, softcap, sink};
#define PM_CASE(K, V) if (kd == K && vd == V) return pm_launch<K, V>(a, B, max_new, stream)
  PM_CASE(64, 64); PM_CASE(64, 128); PM_CASE(96, 64); PM_CASE(96, 128); PM_CASE(128, 64); PM_CASE(128, 128);
  PM_CASE(192, 64); PM_CASE(192, 128); PM_CASE(256, 64); PM_CASE(256, 128);
#undef PM_CASE
  return SLLM_ERR_ARG;
}
