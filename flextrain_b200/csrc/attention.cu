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
// in TMEM across the loop (deterministic), dQ is accumulated with fp32 atomics into a workspace and converted.
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
  int causal;
  int window;             // 0 = unlimited
};

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

template <int HD>
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
      const float m_new = fmaxf(m, mx * c);
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
          pr[i] = keep ? exp2f(__uint_as_float(v[i]) * c - mref) : 0.f;
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

template <int HD>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                      int tiles, cudaStream_t s) {
  constexpr int SMEM = TQ * HD * 2 + 4 * TK * HD * 2 + TQ * TK * 2 + 256 + 1024;
  auto kern = fa_fwd_kernel<HD>;
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

}  // namespace ftb

using namespace ftb;

extern "C" {

// q (Tq, H, hd), k / v (Tk, KV, hd) bf16 with token strides (elements) q_stride / k_stride / v_stride;
// out (Tq, H, hd) contiguous; lse (H, Tq) fp32. cu_q / cu_k: device int32 (num_seqs + 1).
// max_tiles >= sum over sequences of ceil(len_q / 128); Tq / 128 + num_seqs always suffices.
int ftb_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q, const int* cu_k,
                 int num_seqs, int total_q, int total_k, int H, int KV, int hd, long q_stride, long k_stride,
                 long v_stride, float scale, int causal, int window, int max_tiles, cudaStream_t stream) {
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
  p.scale = scale; p.causal = causal; p.window = window;
  if (hd == 128) return launch_fwd<128>(tq, tk, tv, p, max_tiles, stream);
  return launch_fwd<64>(tq, tk, tv, p, max_tiles, stream);
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
