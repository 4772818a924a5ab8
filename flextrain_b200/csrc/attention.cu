// Flash attention for sm_100a on tcgen05 / TMEM: varlen, GQA, causal with bottom-right alignment (the Lq queries
// of a sequence are the last Lq positions of its Lk keys, which is what a chunk of a long sequence sees), optional
// sliding window.  Replaces the external flash-attn 2/3/4 wheels the reference dispatches to
// (flextrain/ops/_kernels/attention.py:180-368, 629-759).
//
// Forward, one CTA per (128-query tile, head):
//   warp 0      TMA producer: Q once, then K / V tiles of 128 keys through two-stage rings (no multicast)
//   warp 1      MMA issuer:   S = Q·Kᵀ into a double-buffered TMEM accumulator, then PV = P·V
//   warps 2-5   softmax:      one query row per thread; S is read from TMEM, P is written as bf16 into a
//                             128B-swizzled shared tile that feeds the second MMA; the running output row
//                             lives in registers (O = O·alpha + PV), so nothing is ever rescaled in TMEM
// S_{j+1} is issued before the softmax of tile j completes, so the tensor core works under the exponentials.
//
// Backward, one CTA per (128-key tile, KV head): loops over the query heads of the group and over the query
// tiles that see these keys; five MMAs per pair (S, dP, dV += Pᵀ·dO, dK += dSᵀ·Q, dQ += dS·K); dK / dV accumulate
// in TMEM across the loop (deterministic).  dQ goes into an fp32 workspace with vector reductions (red.v4.f32) issued
// straight from the registers that hold the tile.  In deterministic mode the CTAs that add to the same (query tile,
// head) take turns in DEscending key-tile order through a counter (the CTA of key tile j adds once the j_hi - j tiles
// above it have added; those reach the query tile earlier in their own loops, so the wait is normally already
// satisfied), which fixes the summation order and makes dQ bit-reproducible.
#include "ptx.cuh"

namespace ftb {

constexpr int FA_THREADS = 192;
constexpr int TQ = 128;   // query rows per tile
constexpr int TK = 128;   // keys per tile

struct FwdParams {
  const int* cu_q;
  const int* cu_k;
  int num_seqs;
  int H, KV;
  __nv_bfloat16* out;     // (Tq, H, HD) contiguous
  float* lse;             // (H, Tq)
  int total_q;
  float scale;
  float softcap;          // 0 = none; else scores become softcap * tanh(scale * s / softcap) (Gemma 2)
  int causal;
  int window;             // 0 = unlimited
};

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ bool find_tile(const int* cu_q, int num_seqs, int tile, int& seq, int& q0) {
  int acc = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int len = cu_q[s + 1] - cu_q[s];
    const int nt = (len + TQ - 1) / TQ;
    if (tile < acc + nt) {
      seq = s;
      q0 = (tile - acc) * TQ;
      return true;
    }
    acc += nt;
  }
  return false;
}

// Byte offset of element (row, col) inside a K-major 128B-swizzled tile made of 64-column blocks of `rows` rows.
__device__ __forceinline__ uint32_t sw128_offset(int row, int col, int rows) {
  const int kb = col >> 6, c = col & 63;
  const int chunk = (c >> 3) ^ (row & 7);
  return static_cast<uint32_t>(kb * rows * 128 + row * 128 + chunk * 16 + (c & 7) * 2);
}

template <int HD, bool CAP>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  constexpr int KB = HD / 64;                 // 64-column blocks of the head dimension
  constexpr int Q_BYTES = TQ * HD * 2;
  constexpr int KV_BYTES = TK * HD * 2;
  constexpr int P_BYTES = TQ * TK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;                 // 2 stages
  uint8_t* sV = sK + 2 * KV_BYTES;            // 2 stages
  uint8_t* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;                    // 1
  uint64_t* k_full = bars + 1;                // 2
  uint64_t* k_empty = bars + 3;               // 2
  uint64_t* v_full = bars + 5;                // 2
  uint64_t* v_empty = bars + 7;               // 2
  uint64_t* s_full = bars + 9;                // 2
  uint64_t* s_empty = bars + 11;              // 2
  uint64_t* p_full = bars + 13;               // 1
  uint64_t* pv_full = bars + 14;              // 1
  uint64_t* pv_empty = bars + 15;             // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kvh = head / (p.H / p.KV);
  int seq = 0, q0 = 0;
  const bool live = find_tile(p.cu_q, p.num_seqs, blockIdx.x, seq, q0);
  if (!live) return;   // uniform for the CTA: nothing allocated yet
  const int qs = p.cu_q[seq], len_q = p.cu_q[seq + 1] - qs;
  const int ks = p.cu_k[seq], len_k = p.cu_k[seq + 1] - ks;
  const int off = len_k - len_q;
  const int rows = min(TQ, len_q - q0);
  int kv_hi = p.causal ? min(len_k, q0 + rows + off) : len_k;
  int kv_lo = (p.causal && p.window > 0) ? max(0, q0 + off - p.window + 1) : 0;
  kv_lo = (kv_lo / TK) * TK;
  const int n_tiles = kv_hi > kv_lo ? (kv_hi - kv_lo + TK - 1) / TK : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4); mbar_init(pv_full, 1); mbar_init(pv_empty, 4);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base;            // 2 x 128 columns
  const uint32_t tm_PV = tmem_base + 256;     // HD columns

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) tma_load_3d(sQ + kb * (TQ * 128), &tmQ, q_full, kb * 64, head, qs + q0);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int key0 = ks + kv_lo + j * TK;
        if (!(ok = mbar_wait(&k_empty[st], ph ^ 1, abort_flag, 110))) break;
        mbar_expect_tx(&k_full[st], KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_3d(sK + st * KV_BYTES + kb * (TK * 128), &tmK, &k_full[st], kb * 64, kvh, key0);
        if (!(ok = mbar_wait(&v_empty[st], ph ^ 1, abort_flag, 111))) break;
        mbar_expect_tx(&v_full[st], KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_3d(sV + st * KV_BYTES + kb * (TK * 128), &tmV, &v_full[st], kb * 64, kvh, key0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(TQ, TK, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TQ, HD, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait(q_full, 0, abort_flag, 120);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, 121)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, abort_flag, 122)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tm_S + st * TK, make_smem_desc(aQ + kb * (TQ * 128) + kk * 32, 16, 1024),
                     make_smem_desc(aK + kb * (TK * 128) + kk * 32, 16, 1024), idesc_s, (kb | kk) != 0);
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          if (!(ok = issue_s(j + 1))) break;
        }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!(ok = mbar_wait(p_full, j & 1, abort_flag, 123))) break;
        if (!(ok = mbar_wait(&v_full[st], ph, abort_flag, 124))) break;
        if (!(ok = mbar_wait(pv_empty, (j & 1) ^ 1, abort_flag, 125))) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + st * KV_BYTES);
#pragma unroll
        for (int s = 0; s < TK / 16; ++s) {
          const uint64_t ad = make_smem_desc(aP + (s >> 2) * (TQ * 128) + (s & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aV + s * (16 * 128), TK * 128, 1024);
          umma_f16(tm_PV, ad, bd, idesc_pv, s != 0);
        }
        umma_commit(pv_full);
        umma_commit(&v_empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // query row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float c = p.scale * 1.4426950408889634f;  // scores are kept in log2 units
    constexpr bool capped = CAP;   // soft-cap is a template parameter: the plain path carries no extra work
    const float cap2 = p.softcap * 1.4426950408889634f;            // soft-cap in log2 units
    const float soc = capped ? p.scale / p.softcap : 0.f;
    float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    const int qi = q0 + r + off;                    // last key this row may see (causal)
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int key0 = kv_lo + j * TK;
      if (!(ok = mbar_wait(&s_full[st], ph, abort_flag, 130))) break;
      tc_fence_after();
      const uint32_t ts = tm_S + st * TK + lane_base;
      // pass 1: row maximum of the masked scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int cb = 0; cb < TK; cb += 32) {
        uint32_t v[32];
        tmem_ld_32x32(ts + cb, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kj = key0 + cb + i;
          bool keep = kj < len_k;
          if (p.causal) keep = keep && (kj <= qi) && (p.window <= 0 || kj > qi - p.window);
          if (keep) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      // tanh is monotonic: the capped maximum is the cap of the maximum
      float m_new;
      if constexpr (CAP) m_new = fmaxf(m, mx == -INFINITY ? mx : cap2 * tanh_fast(mx * soc));
      else m_new = fmaxf(m, mx * c);
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      // fold the previous tile's P·V into the running output (this also means the P tile is free again)
      if (j > 0) {
        if (!(ok = mbar_wait(pv_full, (j - 1) & 1, abort_flag, 131))) break;
        tc_fence_after();
#pragma unroll
        for (int cb = 0; cb < HD; cb += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tm_PV + lane_base + cb, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[cb + i] = o[cb + i] * alpha_prev + __uint_as_float(v[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pv_empty);
      }
      // pass 2: probabilities -> bf16 -> swizzled shared tile; row sum
      float sum = 0.f;
      const float mref = (m_new == -INFINITY) ? 0.f : m_new;
#pragma unroll 1
      for (int cb = 0; cb < TK; cb += 32) {
        uint32_t v[32];
        tmem_ld_32x32(ts + cb, v);
        tmem_ld_wait();
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kj = key0 + cb + i;
          bool keep = kj < len_k;
          if (p.causal) keep = keep && (kj <= qi) && (p.window <= 0 || kj > qi - p.window);
          // two textually separate forms: the plain one must stay a single multiply-add feeding the exponential
          if constexpr (CAP) pr[i] = keep ? exp2f(cap2 * tanh_fast(__uint_as_float(v[i]) * soc) - mref) : 0.f;
          else pr[i] = keep ? exp2f(__uint_as_float(v[i]) * c - mref) : 0.f;
          sum += pr[i];
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 pk;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(pr[g * 8 + 2 * e], pr[g * 8 + 2 * e + 1]);
          *reinterpret_cast<uint4*>(sP + sw128_offset(r, cb + g * 8, TQ)) = pk;
        }
      }
      l = l * alpha + sum;
      m = m_new;
      alpha_prev = alpha;
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[st]);
        mbar_arrive(p_full);
      }
    }
    if (ok && n_tiles > 0) {
      if (mbar_wait(pv_full, (n_tiles - 1) & 1, abort_flag, 132)) {
        tc_fence_after();
#pragma unroll
        for (int cb = 0; cb < HD; cb += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tm_PV + lane_base + cb, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[cb + i] = o[cb + i] * alpha_prev + __uint_as_float(v[i]);
        }
      }
    }
    if (r < rows) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t row = static_cast<size_t>(qs + q0 + r);
      __nv_bfloat16* dst = p.out + (row * p.H + head) * HD;
#pragma unroll
      for (int i = 0; i < HD; i += 8) {
        uint4 pk;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(o[i + 2 * e] * inv, o[i + 2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(dst + i) = pk;
      }
      // natural-log LSE of the scaled scores
      p.lse[static_cast<size_t>(head) * p.total_q + row] = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// =====================================================================================================
// Forward, two query tiles per CTA (the default).  A CTA owns 256 consecutive query rows of one head as two 128-row
// tiles that share every K / V tile (half the K / V traffic of one tile per CTA) and run in ping-pong: while the four
// softmax warps of one tile work on their scores, the tensor core computes the other tile's S = Q·Kᵀ or O += P·V.
//   warps 0-3   softmax of tile 0        warps 4-7   softmax of tile 1
//   warp 8      TMA producer (Q tiles once, K / V through two-stage rings, no multicast)
//   warp 9      MMA issuer
// Tensor memory: S0 | S1 | O0 | O1 (4 x 128 columns).  The probabilities never touch shared memory: a softmax thread
// writes its row of P as packed bf16 over the first 64 columns of its S (tcgen05.st; the write position trails the
// read position of the second pass) and the P·V MMA takes its A operand from tensor memory.  O accumulates in tensor
// memory across the K / V tiles; it is rescaled only when a row maximum has grown by more than 2^8 since the last
// rescale (the probabilities are computed against that stale maximum, so they stay below 2^8 and the final division
// by the row sum is exact), which for real score distributions happens on the first tiles of a row only.
// =====================================================================================================
constexpr int FA2_THREADS = 320;
constexpr float FA2_RESCALE_LOG2 = 8.0f;

__device__ __forceinline__ bool find_tile2(const int* cu_q, int num_seqs, int tile, int& seq, int& q0) {
  int acc = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int len = cu_q[s + 1] - cu_q[s];
    const int nt = (len + 2 * TQ - 1) / (2 * TQ);
    if (tile < acc + nt) {
      seq = s;
      q0 = (tile - acc) * 2 * TQ;
      return true;
    }
    acc += nt;
  }
  return false;
}

template <int HD, bool CAP>
__global__ void __launch_bounds__(FA2_THREADS, 1)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  constexpr int KB = HD / 64;
  constexpr int Q_BYTES = TQ * HD * 2;
  constexpr int KV_BYTES = TK * HD * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                         // 2 tiles
  uint8_t* sK = sQ + 2 * Q_BYTES;             // 2 stages
  uint8_t* sV = sK + 2 * KV_BYTES;            // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * KV_BYTES);
  uint64_t* q_full = bars;                    // 1
  uint64_t* k_full = bars + 1;                // 2
  uint64_t* k_empty = bars + 3;               // 2
  uint64_t* v_full = bars + 5;                // 2
  uint64_t* v_empty = bars + 7;               // 2
  uint64_t* s_full = bars + 9;                // 2 (per query tile)
  uint64_t* p_full = bars + 11;               // 2
  uint64_t* o_full = bars + 13;               // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kvh = head / (p.H / p.KV);
  int seq = 0, q0 = 0;
  // Blocks are handed out in increasing blockIdx; walking the tiles backwards puts the late query blocks of a sequence
  // (the ones with the most K / V tiles under a causal mask) first and leaves the short ones for the tail of the grid.
  if (!find_tile2(p.cu_q, p.num_seqs, static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x), seq, q0))
    return;                                                            // uniform for the CTA: nothing allocated yet
  const int qs = p.cu_q[seq], len_q = p.cu_q[seq + 1] - qs;
  const int ks = p.cu_k[seq], len_k = p.cu_k[seq + 1] - ks;
  const int off = len_k - len_q;
  int kv_lo = (p.causal && p.window > 0) ? max(0, q0 + off - p.window + 1) : 0;
  kv_lo = (kv_lo / TK) * TK;
  // per query tile: live rows and K / V tiles it has to visit (scalars: no indexed local arrays)
  const int rows0 = max(0, min(TQ, len_q - q0)), rows1 = max(0, min(TQ, len_q - q0 - TQ));
  const int hi0 = rows0 == 0 ? 0 : (p.causal ? min(len_k, q0 + rows0 + off) : len_k);
  const int hi1 = rows1 == 0 ? 0 : (p.causal ? min(len_k, q0 + TQ + rows1 + off) : len_k);
  const int nt0 = hi0 > kv_lo ? (hi0 - kv_lo + TK - 1) / TK : 0;
  const int nt1 = hi1 > kv_lo ? (hi1 - kv_lo + TK - 1) / TK : 0;
  const int n_max = max(nt0, nt1);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_full[i], 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------------------- TMA producer
    if (lane == 0 && n_max > 0) {
      const int nq = rows1 > 0 ? 2 : 1;
      mbar_expect_tx(q_full, nq * Q_BYTES);
      for (int t = 0; t < nq; ++t)
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_3d(sQ + t * Q_BYTES + kb * (TQ * 128), &tmQ, q_full, kb * 64, head, qs + q0 + t * TQ);
      bool ok = true;
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int key0 = ks + kv_lo + j * TK;
        if (!(ok = mbar_wait(&k_empty[st], ph ^ 1, abort_flag, 140))) break;
        mbar_expect_tx(&k_full[st], KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_3d(sK + st * KV_BYTES + kb * (TK * 128), &tmK, &k_full[st], kb * 64, kvh, key0);
        if (!(ok = mbar_wait(&v_empty[st], ph ^ 1, abort_flag, 141))) break;
        mbar_expect_tx(&v_full[st], KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_3d(sV + st * KV_BYTES + kb * (TK * 128), &tmV, &v_full[st], kb * 64, kvh, key0);
      }
    }
  } else if (warp == 9) {
    // --------------------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_max > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(TQ, TK, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(TQ, HD, 0, 1);
      bool ok = mbar_wait(q_full, 0, abort_flag, 150);
      // S_t(j) = Q_t · K_jᵀ into the tile's score columns (they are free: the tile's P·V of j-1 was issued before)
      auto issue_s = [&](int t, int j) {
        const uint32_t aQ = smem_u32(sQ + t * Q_BYTES), aK = smem_u32(sK + (j & 1) * KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + t * TK, make_smem_desc(aQ + kb * (TQ * 128) + kk * 32, 16, 1024),
                     make_smem_desc(aK + kb * (TK * 128) + kk * 32, 16, 1024), idesc_s, (kb | kk) != 0);
        umma_commit(&s_full[t]);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, 151);
      if (ok) {
        tc_fence_after();
        if (nt0 > 0) issue_s(0, 0);
        if (nt1 > 0) issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const bool more = j + 1 < n_max;
        if (!(ok = mbar_wait(&v_full[st], ph, abort_flag, 152))) break;
        if (more && !(ok = mbar_wait(&k_full[st ^ 1], ((j + 1) >> 1) & 1, abort_flag, 153))) break;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const int nt = t ? nt1 : nt0;
          if (!ok || j >= nt) continue;
          if (!(ok = mbar_wait(&p_full[t], j & 1, abort_flag, 154 + t))) break;
          tc_fence_after();
          const uint32_t aV = smem_u32(sV + st * KV_BYTES);
#pragma unroll
          for (int s2 = 0; s2 < TK / 16; ++s2)       // P (tensor memory, 8 columns per 16 keys) times V
            umma_f16_ts(tmem_base + 256 + t * HD, tmem_base + t * TK + s2 * 8,
                        make_smem_desc(aV + s2 * (16 * 128), TK * 128, 1024), idesc_pv, (j | s2) != 0);
          umma_commit(&o_full[t]);
          if (j + 1 < nt) issue_s(t, j + 1);
        }
        if (!ok) break;
        umma_commit(&v_empty[st]);
        if (more) umma_commit(&k_empty[st ^ 1]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output of tile t
    const int t = warp >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;                 // query row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tm_S = tmem_base + t * TK + lane_base;
    const uint32_t tm_O = tmem_base + 256 + t * HD + lane_base;
    const float c = p.scale * 1.4426950408889634f;  // scores are kept in log2 units
    const float cap2 = p.softcap * 1.4426950408889634f;
    const float soc = CAP ? p.scale / p.softcap : 0.f;
    const int n_tiles = t ? nt1 : nt0;
    const int rows = t ? rows1 : rows0;
    const int tq0 = q0 + t * TQ;
    const int qi = tq0 + r + off;                   // last key this row may see (causal)
    float m = -INFINITY, l = 0.f;                   // m: the maximum the probabilities are currently scaled against
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int key0 = kv_lo + j * TK;
      if (!(ok = mbar_wait(&s_full[t], j & 1, abort_flag, 160 + t))) break;
      tc_fence_after();
      // The whole score row of this tile goes into registers with one wait (four loads in flight), so tensor memory
      // is read once.  Only tiles that cross the causal diagonal, the window edge or the end of the keys pay for
      // masking (a masked score becomes -inf, whose exponential is 0); interior tiles run the bare
      // max / multiply-add / exp2 / pack stream.
      uint32_t sv[4][32];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) tmem_ld_32x32(tm_S + q4 * 32, sv[q4]);
      tmem_ld_wait();
      const bool edge = (key0 + TK > len_k) ||
                        (p.causal && (key0 + TK - 1 > tq0 + off || (p.window > 0 && key0 <= tq0 + TQ - 1 + off - p.window)));
      if (edge) {
        // visible columns of this row inside the tile: [lo, hi] (one subtract and one unsigned compare per element)
        const int hi = (p.causal ? min(len_k - 1, qi) : len_k - 1) - key0;
        const int lo = (p.causal && p.window > 0) ? max(0, qi - p.window + 1 - key0) : 0;
        const unsigned span = hi >= lo ? static_cast<unsigned>(hi - lo) : 0u;
        const bool none = hi < lo;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (none || static_cast<unsigned>(q4 * 32 + i - lo) > span) sv[q4][i] = 0xff800000u;   // -inf
      }
      float mx4[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        float a = __uint_as_float(sv[q4][0]);
#pragma unroll
        for (int i = 1; i < 32; ++i) a = fmaxf(a, __uint_as_float(sv[q4][i]));
        mx4[q4] = a;
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float m_new;
      if constexpr (CAP) m_new = fmaxf(m, mx == -INFINITY ? mx : cap2 * tanh_fast(mx * soc));
      else m_new = fmaxf(m, mx * c);
      if (j == 0) {
        m = m_new;
      } else {
        const bool grow = m_new > m + FA2_RESCALE_LOG2;
        if (__any_sync(0xffffffffu, grow)) {
          // the tile's previous P·V must have landed before its output rows are rescaled in tensor memory
          if (!(ok = mbar_wait(&o_full[t], (j - 1) & 1, abort_flag, 162 + t))) break;
          tc_fence_after();
          const float alpha = grow ? exp2f(m - m_new) : 1.f;
#pragma unroll 1
          for (int cb = 0; cb < HD; cb += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tm_O + cb, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(tm_O + cb, v);
          }
          tmem_st_wait();
          l *= alpha;
          if (grow) m = m_new;
        }
      }
      // probabilities against m -> packed bf16 over the first half of this tile's S columns; row sum
      const float mref = (m == -INFINITY) ? 0.f : m;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0, p1;
          // two textually separate forms: the plain one must stay a single multiply-add feeding the exponential
          if constexpr (CAP) {
            const float s0 = __uint_as_float(sv[q4][i]), s1 = __uint_as_float(sv[q4][i + 1]);
            p0 = s0 == -INFINITY ? 0.f : exp2f(cap2 * tanh_fast(s0 * soc) - mref);
            p1 = s1 == -INFINITY ? 0.f : exp2f(cap2 * tanh_fast(s1 * soc) - mref);
          } else {
            p0 = exp2f(__uint_as_float(sv[q4][i]) * c - mref);
            p1 = exp2f(__uint_as_float(sv[q4][i + 1]) * c - mref);
          }
          sum4[q4] += p0 + p1;
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
          pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        tmem_st_32x16(tm_S + q4 * 16, pk);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l += sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    if (ok && n_tiles > 0 && mbar_wait(&o_full[t], (n_tiles - 1) & 1, abort_flag, 164 + t)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t row = static_cast<size_t>(qs + tq0 + min(r, max(rows - 1, 0)));
      __nv_bfloat16* dst = p.out + (row * p.H + head) * HD;
#pragma unroll 1
      for (int cb = 0; cb < HD; cb += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tm_O + cb, v);
        tmem_ld_wait();
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o4;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              h2[e] = __floats2bfloat162_rn(__uint_as_float(v[i + 2 * e]) * inv, __uint_as_float(v[i + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + cb + i) = o4;
          }
        }
      }
      // natural-log LSE of the scaled scores
      if (r < rows)
        p.lse[static_cast<size_t>(head) * p.total_q + row] = (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    } else if (n_tiles == 0 && r < rows) {
      // no visible key at all (cannot happen with causal bottom-right alignment, kept for completeness)
      const size_t row = static_cast<size_t>(qs + tq0 + r);
      __nv_bfloat16* dst = p.out + (row * p.H + head) * HD;
      for (int i = 0; i < HD; i += 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
      p.lse[static_cast<size_t>(head) * p.total_q + row] = -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// (rows, heads, hd) bf16 tensor with token stride `row_stride` elements; box = 64 x 1 x box_rows.
static int make_tmap_3d(CUtensorMap* out, const void* base, int hd, int heads, long rows, long row_stride,
                        int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -100;
  cuuint64_t gdim[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)rows};
  cuuint64_t gstr[2] = {(cuuint64_t)hd * 2, (cuuint64_t)row_stride * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -200 - static_cast<int>(r);
}

template <int HD, bool CAP>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                      int tiles, cudaStream_t s) {
  constexpr int SMEM = TQ * HD * 2 + 4 * TK * HD * 2 + TQ * TK * 2 + 256 + 1024;
  auto kern = fa_fwd_kernel<HD, CAP>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -300 - static_cast<int>(e);
    configured = true;
  }
  dim3 grid(tiles, p.H);
  kern<<<grid, FA_THREADS, SMEM, s>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - static_cast<int>(e);
}

template <int HD, bool CAP>
static int launch_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                       int tiles, cudaStream_t s) {
  constexpr int SMEM = 2 * TQ * HD * 2 + 4 * TK * HD * 2 + 256 + 1024;
  auto kern = fa_fwd2_kernel<HD, CAP>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -300 - static_cast<int>(e);
    configured = true;
  }
  dim3 grid(tiles, p.H);
  kern<<<grid, FA2_THREADS, SMEM, s>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - static_cast<int>(e);
}

}  // namespace ftb

using namespace ftb;

static int g_fwd_two_tiles = 1;     // ftb_attn_set_two_tiles(0) selects the one-tile-per-CTA forward kernel

extern "C" {

void ftb_attn_set_two_tiles(int on) { g_fwd_two_tiles = on; }

// q (Tq, H, hd), k / v (Tk, KV, hd) bf16 with token strides (elements) q_stride / k_stride / v_stride;
// out (Tq, H, hd) contiguous; lse (H, Tq) fp32. cu_q / cu_k: device int32 (num_seqs + 1).
// max_tiles >= sum over sequences of ceil(len_q / 128); Tq / 128 + num_seqs always suffices.
int ftb_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q, const int* cu_k,
                 int num_seqs, int total_q, int total_k, int H, int KV, int hd, long q_stride, long k_stride,
                 long v_stride, float scale, float softcap, int causal, int window, int max_tiles,
                 cudaStream_t stream) {
  if (total_q <= 0 || num_seqs <= 0) return 0;
  if ((hd != 64 && hd != 128) || H % KV) return -2;
  if ((q_stride & 7) || (k_stride & 7) || (v_stride & 7)) return -2;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_3d(&tq, q, hd, H, total_q, q_stride, TQ);
  if (rc) return rc;
  rc = make_tmap_3d(&tk, k, hd, KV, total_k, k_stride, TK);
  if (rc) return rc;
  rc = make_tmap_3d(&tv, v, hd, KV, total_k, v_stride, TK);
  if (rc) return rc;
  FwdParams p;
  p.cu_q = cu_q; p.cu_k = cu_k; p.num_seqs = num_seqs; p.H = H; p.KV = KV;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse; p.total_q = total_q;
  p.scale = scale; p.softcap = softcap; p.causal = causal; p.window = window;
  if (g_fwd_two_tiles) {
    const int tiles2 = (total_q + 2 * TQ - 1) / (2 * TQ) + num_seqs;   // >= sum over sequences of ceil(len_q / 256)
    if (softcap > 0.f)
      return hd == 128 ? launch_fwd2<128, true>(tq, tk, tv, p, tiles2, stream)
                       : launch_fwd2<64, true>(tq, tk, tv, p, tiles2, stream);
    return hd == 128 ? launch_fwd2<128, false>(tq, tk, tv, p, tiles2, stream)
                     : launch_fwd2<64, false>(tq, tk, tv, p, tiles2, stream);
  }
  if (softcap > 0.f)
    return hd == 128 ? launch_fwd<128, true>(tq, tk, tv, p, max_tiles, stream)
                     : launch_fwd<64, true>(tq, tk, tv, p, max_tiles, stream);
  return hd == 128 ? launch_fwd<128, false>(tq, tk, tv, p, max_tiles, stream)
                   : launch_fwd<64, false>(tq, tk, tv, p, max_tiles, stream);
}

int ftb_attn_error(void) {
  int h[2] = {0, 0};
  cudaMemcpyFromSymbol(&h[0], g_error_word, sizeof(int));
  cudaMemcpyFromSymbol(&h[1], g_error_where, sizeof(int));
  if (h[0] != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_error_word, &z, sizeof(int));
    cudaMemcpyToSymbol(g_error_where, &z, sizeof(int));
  }
  return h[0] * 1000 + h[1];
}

}  // extern "C"

static int g_dq_bulk = 1;     // ftb_attn_set_dq_bulk(0): per-thread vector reductions (the earlier drain), for A/B runs

// =====================================================================================================
// Backward
// =====================================================================================================
namespace ftb {

struct BwdParams {
  const int* cu_q;
  const int* cu_k;
  int num_seqs;
  int H, KV;
  float* dq_acc;            // (Tq, H, HD) fp32, zero-initialised by the caller
  int* dq_sem;              // deterministic mode: one counter per (query tile, head), zeroed by the caller; else NULL
  int dq_bulk;              // 1: dQ tiles leave through shared memory as tiled reduce-adds; 0: per-thread vector reductions
  __nv_bfloat16* dk;        // (Tk, KV, HD) contiguous
  __nv_bfloat16* dv;
  const float* lse;         // (H, Tq)
  const float* delta;       // (H, Tq)  rowsum(dO * O)
  int total_q;
  float scale;
  float softcap;
  int causal;
  int window;
};

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ dout, long do_stride, const __nv_bfloat16* __restrict__ out,
                                long o_stride, float* __restrict__ delta, int T, int H, int hd) {
  const long w = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long)T * H) return;
  const int t = (int)(w / H), h = (int)(w % H), lane = threadIdx.x & 31;
  const __nv_bfloat16* a = dout + (size_t)t * do_stride + (size_t)h * hd;
  const __nv_bfloat16* b = out + (size_t)t * o_stride + (size_t)h * hd;
  float s = 0.f;
  for (int i = lane * 2; i < hd; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + i));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[(size_t)h * T + t] = s;
}

// Backward thread layout: warp 0 TMA, warp 1 MMA, warps 2-9 softmax / drain.  Warps w and w + 4 share a tensor-memory
// lane quadrant (rows) and split the columns of every tile between them, so two warps per scheduler work on the
// P / dS tile instead of one.
constexpr int FAB_THREADS = 320;

template <int HD, bool CAP>
__global__ void __launch_bounds__(FAB_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
              const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
              const __grid_constant__ CUtensorMap tmDQ, const BwdParams p) {
  constexpr int KB = HD / 64;
  constexpr int T_BYTES = 128 * HD * 2;       // one Q / dO / K / V tile
  constexpr int P_BYTES = 128 * 128 * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + T_BYTES;
  uint8_t* sQ = sV + T_BYTES;
  uint8_t* sDO = sQ + T_BYTES;
  uint8_t* sP = sDO + T_BYTES;
  uint8_t* sDS = sP + P_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + P_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_full = bars + 4;
  uint64_t* dq_full = bars + 5;
  uint64_t* dq_empty = bars + 6;
  uint64_t* stage_bar = bars + 7;
  uint64_t* drain_bar = bars + 9;          // (bars + 8 holds the tensor-memory slot and the abort flag)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y;
  const int rep = p.H / p.KV;
  int seq = 0, k0 = 0;
  // Blocks are handed out in increasing blockIdx.  Unordered dQ: ascending key tiles, so the causal key tiles with the
  // most query tiles start first.  Ordered dQ: DEscending key tiles, so every CTA only ever waits for CTAs that were
  // handed out before it (a CTA that waited for a later one could fill the GPU with waiters and starve it).
  const int tile_x = p.dq_sem != nullptr ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)
                                         : static_cast<int>(blockIdx.x);
  if (!find_tile(p.cu_k, p.num_seqs, tile_x, seq, k0)) return;
  const int qs = p.cu_q[seq], len_q = p.cu_q[seq + 1] - qs;
  const int ks = p.cu_k[seq], len_k = p.cu_k[seq + 1] - ks;
  const int off = len_k - len_q;
  const int kr = min(128, len_k - k0);
  int i_lo = p.causal ? max(0, k0 - off) : 0;
  int i_hi = (p.causal && p.window > 0) ? min(len_q, k0 + kr + p.window - 1 - off) : len_q;
  i_lo = (i_lo / 128) * 128;
  const int n_qt = i_hi > i_lo ? (i_hi - i_lo + 127) / 128 : 0;
  const int n_iter = n_qt * rep;
  int qtile_base = 0;                                   // index of this sequence's first query tile (semaphores)
  if (p.dq_sem != nullptr)
    for (int s2 = 0; s2 < seq; ++s2) qtile_base += (p.cu_q[s2 + 1] - p.cu_q[s2] + 127) / 128;
  const int n_kt = (len_k + 127) / 128;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(qdo_empty, 1); mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8); mbar_init(dq_full, 1); mbar_init(dq_empty, 8); mbar_init(stage_bar, 8);
    mbar_init(drain_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base, tm_dP = tmem_base + 128, tm_dV = tmem_base + 256, tm_dK = tmem_base + 256 + HD;
  const uint32_t tm_dQ = tm_S;   // dQ reuses the S columns once the softmax warps have consumed S

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(kv_full, 2 * T_BYTES);
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        tma_load_3d(sK + kb * (128 * 128), &tmK, kv_full, kb * 64, kvh, ks + k0);
        tma_load_3d(sV + kb * (128 * 128), &tmV, kv_full, kb * 64, kvh, ks + k0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int h = kvh * rep + it / n_qt;
        const int qt = i_lo + (it % n_qt) * 128;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, abort_flag, 210)) break;
        mbar_expect_tx(qdo_full, 2 * T_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          tma_load_3d(sQ + kb * (128 * 128), &tmQ, qdo_full, kb * 64, h, qs + qt);
          tma_load_3d(sDO + kb * (128 * 128), &tmDO, qdo_full, kb * 64, h, qs + qt);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t id_s = make_idesc_bf16(128, 128, 0, 0);       // S, dP: both operands K-major
      constexpr uint32_t id_t = make_idesc_bf16(128, HD, 1, 1);        // dV, dK: transposed A, MN-major B
      constexpr uint32_t id_q = make_idesc_bf16(128, HD, 0, 1);        // dQ: K-major A, MN-major B
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sDO);
      const uint32_t aP = smem_u32(sP), aDS = smem_u32(sDS);
      bool ok = mbar_wait(kv_full, 0, abort_flag, 220);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!(ok = mbar_wait(qdo_full, ph, abort_flag, 221))) break;
        if (!(ok = mbar_wait(dq_empty, ph ^ 1, abort_flag, 222))) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t o = kb * (128 * 128) + kk * 32;
            umma_f16(tm_S, make_smem_desc(aQ + o, 16, 1024), make_smem_desc(aK + o, 16, 1024), id_s, (kb | kk) != 0);
          }
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t o = kb * (128 * 128) + kk * 32;
            umma_f16(tm_dP, make_smem_desc(aDO + o, 16, 1024), make_smem_desc(aV + o, 16, 1024), id_s, (kb | kk) != 0);
          }
        umma_commit(sdp_full);
        if (!(ok = mbar_wait(pds_full, ph, abort_flag, 223))) break;
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 8; ++s) {      // reduction over the 128 query rows, 16 per step
          const uint32_t o = s * (16 * 128);
          umma_f16(tm_dV, make_smem_desc(aP + o, 128 * 128, 1024), make_smem_desc(aDO + o, 128 * 128, 1024), id_t,
                   (it | s) != 0);
          umma_f16(tm_dK, make_smem_desc(aDS + o, 128 * 128, 1024), make_smem_desc(aQ + o, 128 * 128, 1024), id_t,
                   (it | s) != 0);
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) {      // reduction over the 128 keys
          const uint64_t ad = make_smem_desc(aDS + (s >> 2) * (128 * 128) + (s & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aK + s * (16 * 128), 128 * 128, 1024);
          umma_f16(tm_dQ, ad, bd, id_q, s != 0);
        }
        umma_commit(dq_full);
        umma_commit(qdo_empty);
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;               // which half of the columns this warp owns
    const int r = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float c = p.scale * 1.4426950408889634f;
    constexpr bool capped = CAP;   // soft-cap is a template parameter: the plain path carries no extra work
    const float cap2 = p.softcap * 1.4426950408889634f;
    const float soc = capped ? p.scale / p.softcap : 0.f;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t ph = it & 1;
      const int h = kvh * rep + it / n_qt;
      const int qt = i_lo + (it % n_qt) * 128;
      const int i = qt + r;
      const bool vq = i < len_q;
      const size_t grow = static_cast<size_t>(qs + (vq ? i : 0));
      const float lse2 = vq ? p.lse[static_cast<size_t>(h) * p.total_q + grow] * 1.4426950408889634f : INFINITY;
      const float dl = vq ? p.delta[static_cast<size_t>(h) * p.total_q + grow] : 0.f;
      const int qi = i + off;
      // a tile needs masking only if it touches the end of the queries / keys, the causal diagonal or the window edge
      const bool edge = (qt + 128 > len_q) || (k0 + 128 > len_k) ||
                        (p.causal && (k0 + 127 > qt + off || (p.window > 0 && k0 <= qt + 127 + off - p.window)));
      if (!(ok = mbar_wait(sdp_full, ph, abort_flag, 230))) break;
      tc_fence_after();
#pragma unroll 1
      for (int cb = half * 64; cb < half * 64 + 64; cb += 32) {
        uint32_t vs[32], vd[32];
        tmem_ld_32x32(tm_S + lane_base + cb, vs);
        tmem_ld_32x32(tm_dP + lane_base + cb, vd);
        tmem_ld_wait();
        float pr[32], ds[32];
        if (edge || capped) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int kj = k0 + cb + e;
            bool keep = vq && kj < len_k;
            if (p.causal) keep = keep && (kj <= qi) && (p.window <= 0 || kj > qi - p.window);
            const float raw = __uint_as_float(vs[e]);
            const float th = capped ? tanh_fast(raw * soc) : 0.f;
            const float pe = keep ? exp2f((capped ? cap2 * th : raw * c) - lse2) : 0.f;
            pr[e] = pe;
            // d(cap * tanh(scale * s / cap)) / ds = scale * (1 - tanh^2)
            ds[e] = pe * (__uint_as_float(vd[e]) - dl) * p.scale * (1.f - th * th);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float pe = exp2f(__uint_as_float(vs[e]) * c - lse2);
            pr[e] = pe;
            ds[e] = pe * (__uint_as_float(vd[e]) - dl) * p.scale;
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 a, b;
          __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a);
          __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            a2[e] = __floats2bfloat162_rn(pr[g * 8 + 2 * e], pr[g * 8 + 2 * e + 1]);
            b2[e] = __floats2bfloat162_rn(ds[g * 8 + 2 * e], ds[g * 8 + 2 * e + 1]);
          }
          const uint32_t o = sw128_offset(r, cb + g * 8, 128);
          *reinterpret_cast<uint4*>(sP + o) = a;
          *reinterpret_cast<uint4*>(sDS + o) = b;
        }
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (!(ok = mbar_wait(dq_full, ph, abort_flag, 231))) break;
      tc_fence_after();
      constexpr int HC = HD / 2;
      if (p.dq_bulk) {
        // dQ tile: tensor memory -> registers -> fp32 staging in shared memory (the P / dS buffers, free now that the
        // MMAs of this query tile are done; one 16 KB block of 128 rows x 32 columns per 32 columns, 128-byte
        // swizzle) -> four (two at hd 64) tiled reduce-adds into the fp32 workspace.  L2 then sees whole 128-byte
        // lines per reduction instead of one 16-byte piece per row and thread, which is what bounded this kernel.
        // Rows past the end of the sequence hold exact zeros (their P and dS were masked), so adding them is harmless.
        uint8_t* stg = sP;
#pragma unroll 1
        for (int cb = half * HC; cb < half * HC + HC; cb += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tm_dQ + lane_base + cb, v);
          tmem_ld_wait();
          uint8_t* rowp = stg + (cb >> 5) * (128 * 128) + r * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(rowp + ((j ^ (r & 7)) << 4)) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(dq_empty);                  // TMEM columns are free: the next S / dP may be issued now
          mbar_arrive(stage_bar);                 // this warp's rows are staged
        }
        if (warp == 2 && lane == 0) {
          bool go = mbar_wait(stage_bar, ph, abort_flag, 232);
          int* sem = nullptr;
          if (go && p.dq_sem != nullptr) {
            // deterministic order: wait until the key tiles above this one have added their share of this query tile
            // (word 0 of the array is the give-up flag, the counters follow it)
            sem = p.dq_sem + 1 + (static_cast<size_t>(qtile_base + qt / 128)) * p.H + h;
            const int j_hi = p.causal ? min(n_kt - 1, (qt + 127 + off) / 128) : n_kt - 1;
            const int expected = j_hi - k0 / 128;
            uint32_t spins = 0;
            volatile int* gave_up = p.dq_sem;
            while (expected > 0 && !*gave_up && ld_acquire_gpu_s32(sem) < expected) {
              if (++spins > (1u << 21) || *abort_flag) { *gave_up = 1; set_error(4, 240); break; }
              __nanosleep(32);
            }
          }
          if (go) {
#pragma unroll
            for (int q4 = 0; q4 < HD / 32; ++q4)
              tma_reduce_add_2d(&tmDQ, stg + q4 * (128 * 128), h * HD + q4 * 32, qs + qt);
            bulk_commit();
            if (sem != nullptr) {
              bulk_wait_all();                    // the additions have been performed: the next key tile may add
              red_release_gpu_add_s32(sem, 1);
            } else {
              bulk_wait_read_all();               // the staging buffers have been read: P / dS may be rewritten
            }
          }
          mbar_arrive(drain_bar);
        }
        if (!(ok = mbar_wait(drain_bar, ph, abort_flag, 233))) break;
        continue;
      }
      // dQ tile: tensor memory -> registers -> vector reductions into the fp32 workspace, one row per thread (eight
      // 16-byte red.v4 per 32 columns).  Each warp drains its own half of the columns of its 32 rows.
      int* sem = nullptr;
      if (p.dq_sem != nullptr) {
        // deterministic order: wait until the key tiles above this one have added their share of this query tile
        // (word 0 of the array is the give-up flag, the counters follow it)
        sem = p.dq_sem + 1 + (static_cast<size_t>(qtile_base + qt / 128)) * p.H + h;
        const int j_hi = p.causal ? min(n_kt - 1, (qt + 127 + off) / 128) : n_kt - 1;
        const int expected = j_hi - k0 / 128;
        if (lane == 0 && expected > 0) {
          uint32_t spins = 0;
          volatile int* gave_up = p.dq_sem;
          while (!*gave_up && ld_acquire_gpu_s32(sem) < expected) {
            // give up: the order is lost, not data.  The flag makes every later wait of this launch return at once,
            // so one lost turn costs one time limit (about a second), not one per tile.
            if (++spins > (1u << 21) || *abort_flag) { *gave_up = 1; set_error(4, 240); break; }
            __nanosleep(32);
          }
        }
        __syncwarp();
      }
      float* dq_row = p.dq_acc + ((static_cast<size_t>(qs + (vq ? i : 0))) * p.H + h) * HD;
#pragma unroll 1
      for (int cb = half * HC; cb < half * HC + HC; cb += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tm_dQ + lane_base + cb, v);
        tmem_ld_wait();
        if (vq) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            red_add_v4_f32(dq_row + cb + e, __uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                           __uint_as_float(v[e + 3]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);       // TMEM columns are free: the next S / dP may be issued now
      if (sem != nullptr) {
        // all eight warps' reductions must be visible before the next key tile in the order may add
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(stage_bar);
        if (!(ok = mbar_wait(stage_bar, ph, abort_flag, 232))) break;
        if (warp == 2 && lane == 0) red_release_gpu_add_s32(sem, 1);
      }
    }
    if (p.dq_bulk && warp == 2 && lane == 0) bulk_wait_all();   // none of this thread's reduce-adds outlives the kernel
    // dK / dV of this key tile (thread = key row)
    constexpr int HC2 = HD / 2;
    if (r < kr) {
      const size_t row = static_cast<size_t>(ks + k0 + r);
      __nv_bfloat16* dk_row = p.dk + (row * p.KV + kvh) * HD;
      __nv_bfloat16* dv_row = p.dv + (row * p.KV + kvh) * HD;
      if (n_iter == 0 || !ok) {
        for (int cidx = half * HC2; cidx < half * HC2 + HC2; cidx += 8) {
          *reinterpret_cast<uint4*>(dk_row + cidx) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dv_row + cidx) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    if (n_iter > 0 && ok) {
      tc_fence_after();
      const size_t row = static_cast<size_t>(ks + k0 + min(r, kr - 1));
      __nv_bfloat16* dk_row = p.dk + (row * p.KV + kvh) * HD;
      __nv_bfloat16* dv_row = p.dv + (row * p.KV + kvh) * HD;
#pragma unroll 1
      for (int cb = half * HC2; cb < half * HC2 + HC2; cb += 32) {
        uint32_t a[32], b[32];
        tmem_ld_32x32(tm_dV + lane_base + cb, a);
        tmem_ld_32x32(tm_dK + lane_base + cb, b);
        tmem_ld_wait();
        if (r < kr) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 x, y;
            __nv_bfloat162* x2 = reinterpret_cast<__nv_bfloat162*>(&x);
            __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&y);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              x2[e] = __floats2bfloat162_rn(__uint_as_float(a[g * 8 + 2 * e]), __uint_as_float(a[g * 8 + 2 * e + 1]));
              y2[e] = __floats2bfloat162_rn(__uint_as_float(b[g * 8 + 2 * e]), __uint_as_float(b[g * 8 + 2 * e + 1]));
            }
            *reinterpret_cast<uint4*>(dv_row + cb + g * 8) = x;
            *reinterpret_cast<uint4*>(dk_row + cb + g * 8) = y;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD, bool CAP>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv,
                      const CUtensorMap& tdq, const BwdParams& p, int tiles, cudaStream_t s) {
  constexpr int SMEM = 4 * 128 * HD * 2 + 2 * 128 * 128 * 2 + 256 + 1024;
  auto kern = fa_bwd_kernel<HD, CAP>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -300 - static_cast<int>(e);
    configured = true;
  }
  dim3 grid(tiles, p.KV);
  kern<<<grid, FAB_THREADS, SMEM, s>>>(tq, tdo, tk, tv, tdq, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - static_cast<int>(e);
}

}  // namespace ftb

extern "C" {

// dout / q / out (Tq, H, hd), k / v (Tk, KV, hd) bf16 with token strides; lse (H, Tq) from the forward.
// Workspaces supplied by the caller: delta (H, Tq) fp32, dq_acc (Tq, H, hd) fp32 ZEROED.
// Outputs: dq (bf16, converted from dq_acc), dk, dv (Tk, KV, hd) bf16 contiguous, every row written.
// dq_sem: NULL, or 1 + (sum over sequences of ceil(len_q / 128)) x H int32 words, ZEROED (word 0 is the kernel's
//   give-up flag, the rest one counter per (query tile, head)): makes the dQ summation order
// fixed (bit-reproducible gradients) at the price of ordering the CTAs that share a query tile.
int ftb_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse,
                 float* delta, float* dq_acc, int* dq_sem, void* dq, void* dk, void* dv, const int* cu_q, const int* cu_k,
                 int num_seqs, int total_q, int total_k, int H, int KV, int hd, long q_stride, long k_stride,
                 long v_stride, long do_stride, long o_stride, float scale, float softcap, int causal, int window,
                 int max_tiles, cudaStream_t stream) {
  if (total_q <= 0 || num_seqs <= 0) return 0;
  if ((hd != 64 && hd != 128) || H % KV) return -2;
  if ((q_stride & 7) || (k_stride & 7) || (v_stride & 7) || (do_stride & 7)) return -2;
  {
    const long warps = (long)total_q * H;
    fa_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)dout, do_stride,
                                                                     (const __nv_bfloat16*)out, o_stride, delta,
                                                                     total_q, H, hd);
  }
  CUtensorMap tq, tdo, tk, tv;
  int rc = make_tmap_3d(&tq, q, hd, H, total_q, q_stride, 128);
  if (rc) return rc;
  rc = make_tmap_3d(&tdo, dout, hd, H, total_q, do_stride, 128);
  if (rc) return rc;
  rc = make_tmap_3d(&tk, k, hd, KV, total_k, k_stride, 128);
  if (rc) return rc;
  rc = make_tmap_3d(&tv, v, hd, KV, total_k, v_stride, 128);
  if (rc) return rc;
  // fp32 workspace as a 2-D tensor (total_q rows of H * hd columns): boxes of 128 rows x 32 columns for the reduce-adds
  CUtensorMap tdq;
  {
    EncodeTiledFn enc = get_encode();
    if (enc == nullptr) return -100;
    cuuint64_t gdim[2] = {(cuuint64_t)H * hd, (cuuint64_t)total_q};
    cuuint64_t gstr[1] = {(cuuint64_t)H * hd * 4};
    cuuint32_t box[2] = {32, 128};
    cuuint32_t es[2] = {1, 1};
    CUresult r = enc(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dq_acc, gdim, gstr, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -200 - static_cast<int>(r);
  }
  BwdParams p;
  p.cu_q = cu_q; p.cu_k = cu_k; p.num_seqs = num_seqs; p.H = H; p.KV = KV; p.dq_bulk = g_dq_bulk;
  p.dq_acc = dq_acc; p.dq_sem = dq_sem; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.lse = lse; p.delta = delta;
  p.total_q = total_q; p.scale = scale; p.softcap = softcap; p.causal = causal; p.window = window;
  if (softcap > 0.f)
    rc = (hd == 128) ? launch_bwd<128, true>(tq, tdo, tk, tv, tdq, p, max_tiles, stream)
                     : launch_bwd<64, true>(tq, tdo, tk, tv, tdq, p, max_tiles, stream);
  else
    rc = (hd == 128) ? launch_bwd<128, false>(tq, tdo, tk, tv, tdq, p, max_tiles, stream)
                     : launch_bwd<64, false>(tq, tdo, tk, tv, tdq, p, max_tiles, stream);
  return rc;
}

// 1 (default): dQ leaves the SM as tiled reduce-adds from shared memory; 0: per-thread vector reductions
void ftb_attn_set_dq_bulk(int on) { g_dq_bulk = on; }

}  // extern "C"
