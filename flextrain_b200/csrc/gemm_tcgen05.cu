// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   D[M,N] = alpha * op(A) * op(B) + beta * C[M,N] (+ bias[N])        fp32 accumulate in TMEM
//
// Replaces the cuBLASLt dispatcher of the reference project
// (helpers/matmul_dispatcher/src/dispatch.cpp:149-322) and its torch.matmul/addmm call sites.
// Structure: persistent, one CTA per SM, warp-specialised
//   warp 0    TMA producer   (cp.async.bulk.tensor 2-D, 128-byte swizzle, no multicast)
//   warp 1    MMA issuer     (tcgen05.mma cta_group::1, 128 x BN x 16 per instruction)
//   warps 2-5 epilogue       (tcgen05.ld 32x32b -> alpha/beta/bias -> global stores)
// with a STAGES-deep shared-memory ring and two TMEM accumulators so the epilogue of tile i
// overlaps the main loop of tile i+1.  Operands may each be K-major or MN-major, which covers
// forward (x·Wᵀ), dgrad (dy·W) and wgrad (dyᵀ·x) with weights kept in (out, in) layout.
//
// A grouped variant (one launch for all experts of an MoE layer, tile list built on the device
// from the expert offsets) shares the same pipeline; see ftb_grouped_gemm_bf16.
#include "ptx.cuh"

namespace ftb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 256;   // warps 0-5: TMA / MMA / epilogue; warps 6-7: peer-panel pull (TP all-gather mode)
constexpr int MAX_RANKS = 8;
constexpr int GROUP_M = 16;  // tile rasterisation: GROUP_M row-tiles share a sweep over N (L2 reuse)

struct GemmParams {
  int M, N, K;
  int ldd, ldc;
  float alpha, beta;
  void* D;
  const void* C;
  const float* bias;
  int d_fp32;        // output (and C) element type: 0 bf16, 1 fp32
  // grouped mode (num_groups > 0): rows of A / D are expert-major, offsets[g]..offsets[g+1];
  // B is (G, N, K) or (G, K, N) addressed through a 3-D tensor map.
  int num_groups;
  const int* offsets;
  int max_tiles;     // grouped: upper bound of tiles the grid walks
  // split-K (plain mode only): the K range is cut into split_k slices of k_per_split elements; slice s of every output
  // tile is a work item of its own and lands in D + s * M * ldd (an fp32 workspace), to be summed by splitk_reduce.
  int split_k, k_per_split;
  // gated-FFN epilogues of the two-SM kernel (EPI 1 / 2, see gemm2_kernel)
  int glu_F, glu_kind;       // F = ffn width (columns of one half); kind 0 SwiGLU, 1 GeGLU(tanh)
  void* glu_act;             // (M, F) bf16: activation output
  int glu_ld_act;
  const void* glu_x13;       // EPI 2: saved forward [gate | up] (M, 2F) bf16
  int glu_ld_x13;
  // ---- tensor-parallel fused modes (comm_mode != 0); rows are split into `world` panels of `panel_rows`
  //  1  all-gather -> GEMM: A's row panel p lives on rank p.  Warps 6-7 of every CTA pull the remote panels
  //     from the peers' staging buffers into the local one (plain peer loads, each byte crosses NVLink once),
  //     publishing bytes-arrived per panel; the TMA producer starts on the local panel and waits per panel.
  //  2  GEMM -> reduce-scatter: output panel p is owned by rank p.  The epilogue stores each partial tile
  //     straight into the owner's staging slot for this rank (peer stores, tile by tile under the math);
  //     a small reduce kernel on the owner then sums the `world` slots.
  int comm_mode, world, rank, panel_rows;
  int pull_threads;          // mode 1: 1 = pull with per-thread 16-byte loads (two warps) instead of bulk copies
  const void* a_peer[MAX_RANKS];
  void* a_local;
  long panel_bytes;
  unsigned long long* panel_counter;
  void* d_peer[MAX_RANKS];
  long d_slot_stride;
  //  3  parameter all-gather -> GEMM (data parallel with the parameter all-gather deferred to first use): B lies in
  //     this rank's parameter arena `a_local`; after the sharded optimizer step only rank r's element range of every
  //     segment is current in r's arena `a_peer[r]`.  Warps 6-7 pull the other ranks' ranges of up to MAX_PULL
  //     segments (the whole layer) into the local arena; `panel_counter[r]` counts the bytes of segment 0 (the one
  //     that holds B) arrived from rank r, and the TMA producer waits for the ranks whose ranges a B tile touches.
  int n_pull, tn_first;
  long pull_off[4], pull_numel[4], pull_per[4];   // byte offset in the arena, elements, elements per rank
  int pull_es[4];                                 // element size in bytes
  long gate_lo;                                   // byte offset of B's first row inside segment 0
};
constexpr int MAX_PULL = 4;

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

// Reduce-scatter epilogue staging: 4 epilogue warps x (32 rows x 128 bf16 columns).
constexpr int RS_STAGE_BYTES = 4 * 32 * 256;
// All-gather mode: two shared-memory buffers of this size carry the remote panels (peer -> shared -> local staging).
constexpr int PULL_CHUNK_BYTES = 16384;

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gm;
  tn = r / gm;
}

// Panel-ordered tiles for the tensor-parallel modes: panels are visited starting at `first`, each panel uses the
// grouped rasterisation internally.
__device__ __forceinline__ void panel_tile_coords(int tile, int tiles_n, int panel_rows, int world, int first,
                                                  int& panel, int& row0, int& tn) {
  const int tiles_m_panel = panel_rows / BM;
  const int per_panel = tiles_m_panel * tiles_n;
  const int pi = tile / per_panel;
  panel = (first + pi) % world;
  int tm;
  tile_coords(tile - pi * per_panel, tiles_m_panel, tiles_n, tm, tn);
  row0 = panel * panel_rows + tm * BM;
}

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Grouped tile lookup: tile index -> (group, row tile inside group). Linear walk over the
// offsets (E <= 256, done by one thread per role per tile; cheap next to a 128xBNxK main loop).
__device__ __forceinline__ bool grouped_tile(const int* __restrict__ offsets, int num_groups, int tiles_n, int tile,
                                             int& g, int& row0, int& rows, int& tn) {
  int acc = 0;
  for (int e = 0; e < num_groups; ++e) {
    const int a = offsets[e], b = offsets[e + 1];
    const int tm_e = (b - a + BM - 1) / BM;
    const int t_e = tm_e * tiles_n;
    if (tile < acc + t_e) {
      const int r = tile - acc;
      g = e;
      const int tm = r % tm_e;
      tn = r / tm_e;
      row0 = a + tm * BM;
      rows = min(BM, b - row0);
      return true;
    }
    acc += t_e;
  }
  return false;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int GROUPED, int COMM = 0>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int splits = (GROUPED == 0 && COMM == 0 && p.split_k > 1) ? p.split_k : 1;
  const int num_tiles = GROUPED == 1 ? p.max_tiles
                                     : (GROUPED == 2 ? p.num_groups * tiles_m * tiles_n : tiles_m * tiles_n * splits);
  int k_blocks = (p.K + BK - 1) / BK;
  // k-blocks of split slice `sp` (all slices but the last are full)
  auto split_blocks = [&](int sp) {
    const int lo = sp * p.k_per_split;
    return (min(p.K, lo + p.k_per_split) - lo + BK - 1) / BK;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    if constexpr (COMM == 1) {           // completion barriers of the two peer-pull buffers
      mbar_init(full_bar + 20, 1);
      mbar_init(full_bar + 21, 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn, g = 0, row0, rows;
        int k_lo = 0;
        if constexpr (GROUPED == 1) {
          if (!grouped_tile(p.offsets, p.num_groups, tiles_n, tile, g, row0, rows, tn)) break;
        } else if constexpr (GROUPED == 2) {
          // per-expert weight gradient: tile = (expert, tm, tn); the reduction runs over the expert's rows
          g = tile / (tiles_m * tiles_n);
          tile_coords(tile - g * tiles_m * tiles_n, tiles_m, tiles_n, tm, tn);
          row0 = tm * BM;
          k_lo = p.offsets[g];
          k_blocks = (p.offsets[g + 1] - k_lo + BK - 1) / BK;
          if (k_blocks == 0) continue;
        } else if constexpr (COMM == 3) {
          tile_coords(tile, tiles_m, tiles_n, tm, tn);
          tn = (tn + p.tn_first) % tiles_n;          // start the sweep over N at the rows this rank owns
          row0 = tm * BM;
          // ranks whose ranges of segment 0 this B tile touches: wait (bounded) for their bytes
          const long rb = p.pull_per[0] * p.pull_es[0];                      // bytes per rank
          const long lo = p.gate_lo + static_cast<long>(tn) * BN * p.K * 2;
          const long hi = min(lo + static_cast<long>(BN) * p.K * 2, p.gate_lo + static_cast<long>(p.N) * p.K * 2);
          for (int r = static_cast<int>(lo / rb); r <= static_cast<int>((hi - 1) / rb) && r < p.world && ok; ++r) {
            if (r == p.rank) continue;
            const long cnt = min(p.pull_numel[0], (r + 1) * p.pull_per[0]) - min(p.pull_numel[0], r * p.pull_per[0]);
            const unsigned long long need = static_cast<unsigned long long>(cnt * p.pull_es[0]);
            uint32_t it = 0;
            while (ld_acquire_gpu_u64(p.panel_counter + r) < need) {
              if (++it > FTB_WAIT_LIMIT || *abort_flag) { *abort_flag = 1; set_error(2, 50 + r); ok = false; break; }
              __nanosleep(64);
            }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        } else if constexpr (COMM != 0) {
          int panel;
          panel_tile_coords(tile, tiles_n, p.panel_rows, p.world, COMM == 1 ? p.rank : p.rank + 1, panel, row0, tn);
          if constexpr (COMM == 1) {
            if (panel != p.rank) {   // wait (bounded) until the pull warps have landed this panel in local memory
              const unsigned long long need = static_cast<unsigned long long>(p.panel_bytes);
              uint32_t it = 0;
              while (ld_acquire_gpu_u64(p.panel_counter + panel) < need) {
                if (++it > FTB_WAIT_LIMIT || *abort_flag) { *abort_flag = 1; set_error(2, 40 + panel); ok = false; break; }
                __nanosleep(64);
              }
              if (!ok) break;
              asm volatile("fence.proxy.async;" ::: "memory");
            }
          }
        } else {
          if (splits > 1) {
            const int sp = tile / (tiles_m * tiles_n);
            tile_coords(tile - sp * tiles_m * tiles_n, tiles_m, tiles_n, tm, tn);
            k_lo = sp * p.k_per_split;
            k_blocks = split_blocks(sp);
          } else {
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
          }
          row0 = tm * BM;
        }
        const int col0 = tn * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 10))) break;
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = k_lo + kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (64 * BK * 2), &tmA, &full_bar[stage], row0 + j * 64, k0);
          }
          if constexpr (GROUPED == 1) {
            if constexpr (!B_MN) {
              tma_load_3d(sb, &tmB, &full_bar[stage], k0, col0, g);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * (64 * BK * 2), &tmB, &full_bar[stage], col0 + j * 64, k0, g);
            }
          } else {
            if constexpr (!B_MN) {
              tma_load_2d(sb, &tmB, &full_bar[stage], k0, col0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (64 * BK * 2), &tmB, &full_bar[stage], col0 + j * 64, k0);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // Drain: wait until every load this thread issued has landed (the consumer may have
      // aborted); bounded, so an unwinding CTA never exits with copies in flight.
      if (!ok) {
        for (int s = 0; s < STAGES; ++s)
          for (uint32_t it = 0; it < (1u << 16); ++it)
            if (mbar_try_wait(&full_bar[s], 0) || mbar_try_wait(&full_bar[s], 1)) break;
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if constexpr (GROUPED == 1) {
          int g, row0, rows, tn;
          if (!grouped_tile(p.offsets, p.num_groups, tiles_n, tile, g, row0, rows, tn)) break;
        }
        if constexpr (GROUPED == 2) {
          const int g = tile / (tiles_m * tiles_n);
          k_blocks = (p.offsets[g + 1] - p.offsets[g] + BK - 1) / BK;
          if (k_blocks == 0) continue;
        }
        if (splits > 1) k_blocks = split_blocks(tile / (tiles_m * tiles_n));
        if (!(ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, 20))) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag, 21))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // K-major: step 32 B inside the 128 B swizzle row. MN-major: step 16 k-rows of 128 B.
            const uint64_t ad = A_MN ? make_smem_desc(sa + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_f16(tmem_d, ad, bd, idesc, (kb | kk) != 0);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);  // accumulator complete -> epilogue
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------- peer pulls (all-gather modes only)
    if constexpr (COMM == 3) {
      const int t = threadIdx.x - 192;                       // 0..63
      const long stride = static_cast<long>(gridDim.x) * 64;
      for (int sgi = 0; sgi < p.n_pull; ++sgi) {
        const long es = p.pull_es[sgi];
        for (int i = 1; i < p.world; ++i) {
          const int r = (p.rank + i) % p.world;
          const long beg = min(p.pull_numel[sgi], r * p.pull_per[sgi]);
          const long cnt = min(p.pull_numel[sgi], (r + 1) * p.pull_per[sgi]) - beg;
          if (cnt <= 0) continue;
          const long off = p.pull_off[sgi] + beg * es;
          const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.a_peer[r]) + off);
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.a_local) + off);
          const long n16 = (cnt * es) >> 4;
          long moved = 0;
          long idx = static_cast<long>(blockIdx.x) * 64 + t;
          for (; idx + 7 * stride < n16; idx += 8 * stride) {   // eight loads in flight per thread
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = src[idx + u * stride];
#pragma unroll
            for (int u = 0; u < 8; ++u) dst[idx + u * stride] = v[u];
            moved += 128;
          }
          for (; idx < n16; idx += stride) { dst[idx] = src[idx]; moved += 16; }
          if (sgi == 0) {
            asm volatile("fence.proxy.async;" ::: "memory");
            __threadfence();
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) moved += __shfl_xor_sync(0xffffffffu, moved, o);
            if (lane == 0 && moved) atomicAdd(p.panel_counter + r, static_cast<unsigned long long>(moved));
          }
        }
      }
    }
    if constexpr (COMM == 1) {
      if (!p.pull_threads) {
        // One thread streams this CTA's share of the remote panels through shared memory with bulk copies:
        // peer memory -> 16 KB buffer (completion on an mbarrier) -> local staging buffer (bulk store).  Two buffers,
        // so each CTA keeps two remote reads in flight (148 CTAs x 32 KB outstanding, enough to cover NVLink latency
        // at full bandwidth) and the copy costs one issuing thread instead of two warps' load/store slots.
        if (warp == 6 && lane == 0) {
          constexpr long CH = PULL_CHUNK_BYTES;
          uint8_t* pbuf = smem + L::BAR_OFFSET + 256;
          uint64_t* pull_bar = full_bar + 20;
          const long per_panel = (p.panel_bytes + CH - 1) / CH;
          const long total = per_panel * (p.world - 1);
          auto locate = [&](long g, int& pn, long& off, uint32_t& n) {
            pn = (p.rank + 1 + static_cast<int>(g / per_panel)) % p.world;
            off = (g % per_panel) * CH;
            n = static_cast<uint32_t>(min(CH, p.panel_bytes - off));
          };
          auto issue = [&](long g, int buf) {
            int pn; long off; uint32_t n;
            locate(g, pn, off, n);
            mbar_expect_tx(&pull_bar[buf], n);
            bulk_load_g2s(pbuf + buf * CH, reinterpret_cast<const char*>(p.a_peer[pn]) + pn * p.panel_bytes + off, n,
                          &pull_bar[buf]);
          };
          auto publish = [&](int pn, long moved) {
            bulk_wait_all();                                   // the panel's stores have been written
            asm volatile("fence.proxy.async;" ::: "memory");
            __threadfence();
            atomicAdd(p.panel_counter + pn, static_cast<unsigned long long>(moved));
          };
          long g = blockIdx.x, moved = 0;
          int k = 0, cur = -1;
          uint32_t phases = 0;
          if (g < total) issue(g, 0);
          for (; g < total; g += gridDim.x, ++k) {
            const int buf = k & 1;
            if (g + gridDim.x < total) {
              bulk_wait_read_all();                            // the other buffer's last store has left shared memory
              issue(g + gridDim.x, buf ^ 1);
            }
            if (!mbar_wait(&pull_bar[buf], (phases >> buf) & 1u, abort_flag, 30)) break;
            phases ^= 1u << buf;
            int pn; long off; uint32_t n;
            locate(g, pn, off, n);
            if (pn != cur && cur >= 0) { publish(cur, moved); moved = 0; }
            cur = pn;
            bulk_store_s2g(reinterpret_cast<char*>(p.a_local) + pn * p.panel_bytes + off, pbuf + buf * CH, n);
            bulk_commit();
            moved += n;
          }
          if (cur >= 0) publish(cur, moved);
          bulk_wait_all();                                     // nothing of this thread's copies outlives the kernel
        }
      } else {
      const int t = threadIdx.x - 192;                       // 0..63
      const long stride = static_cast<long>(gridDim.x) * 64;
      const long n16 = p.panel_bytes >> 4;
      for (int i = 1; i < p.world; ++i) {
        const int pn = (p.rank + i) % p.world;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(p.a_peer[pn]) + pn * p.panel_bytes);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(p.a_local) + pn * p.panel_bytes);
        long moved = 0;
        long idx = static_cast<long>(blockIdx.x) * 64 + t;
        for (; idx + 7 * stride < n16; idx += 8 * stride) {   // eight loads in flight per thread
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = src[idx + u * stride];
#pragma unroll
          for (int u = 0; u < 8; ++u) dst[idx + u * stride] = v[u];
          moved += 128;
        }
        for (; idx < n16; idx += stride) { dst[idx] = src[idx]; moved += 16; }
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) moved += __shfl_xor_sync(0xffffffffu, moved, o);
        if (lane == 0 && moved) atomicAdd(p.panel_counter + pn, static_cast<unsigned long long>(moved));
      }
      }
    }
  } else {
    // ----------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn, g = 0, row0, rows;
      char* d_base = reinterpret_cast<char*>(p.D);
      long d_row_shift = 0;
      if constexpr (GROUPED == 1) {
        if (!grouped_tile(p.offsets, p.num_groups, tiles_n, tile, g, row0, rows, tn)) break;
      } else if constexpr (GROUPED == 2) {
        g = tile / (tiles_m * tiles_n);
        tile_coords(tile - g * tiles_m * tiles_n, tiles_m, tiles_n, tm, tn);
        row0 = tm * BM;
        rows = min(BM, p.M - row0);
        if ((p.offsets[g + 1] - p.offsets[g] + BK - 1) / BK == 0) continue;   // empty expert: gradient unchanged
        d_base = reinterpret_cast<char*>(p.D) + static_cast<size_t>(g) * p.M * p.ldd * (p.d_fp32 ? 4 : 2);
      } else if constexpr (COMM == 3) {
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        tn = (tn + p.tn_first) % tiles_n;
        row0 = tm * BM;
        rows = min(BM, p.M - row0);
      } else if constexpr (COMM != 0) {
        int panel;
        panel_tile_coords(tile, tiles_n, p.panel_rows, p.world, COMM == 1 ? p.rank : p.rank + 1, panel, row0, tn);
        rows = BM;
        if constexpr (COMM == 2) {   // partial tile goes to the owner's slot for this rank
          d_base = reinterpret_cast<char*>(p.d_peer[panel]) +
                   static_cast<size_t>(p.rank) * p.d_slot_stride * (p.d_fp32 ? 4 : 2);
          d_row_shift = static_cast<long>(panel) * p.panel_rows;
        }
      } else {
        if (splits > 1) {
          const int sp = tile / (tiles_m * tiles_n);
          tile_coords(tile - sp * tiles_m * tiles_n, tiles_m, tiles_n, tm, tn);
          d_base = reinterpret_cast<char*>(p.D) + static_cast<size_t>(sp) * p.M * p.ldd * 4;   // fp32 slice
        } else {
          tile_coords(tile, tiles_m, tiles_n, tm, tn);
        }
        row0 = tm * BM;
        rows = min(BM, p.M - row0);
      }
      if (!(ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, 30))) break;
      tc_fence_after();
      const int r_in = quad * 32 + lane;
      const bool row_ok = r_in < rows;
      const size_t row = static_cast<size_t>(row0 + r_in - d_row_shift);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if constexpr (COMM == 2) {
        // Peer stores: a lane-per-row store puts 16 B per row on the wire per instruction.  Stage 32 rows x 128
        // columns per warp in shared memory (16-byte chunks XOR-swizzled by row) and write whole 256-byte row
        // segments, 16 lanes per row, so every NVLink write request carries a full segment.
        if (!p.d_fp32) {
          uint8_t* stg = smem + L::BAR_OFFSET + 256 + quad * (RS_STAGE_BYTES / 4);
          __nv_bfloat16* dmat = reinterpret_cast<__nv_bfloat16*>(d_base);
#pragma unroll 1
          for (int half = 0; half < BN; half += 128) {
            const int col_h = tn * BN + half;
            if (col_h >= p.N) break;
#pragma unroll 1
            for (int c = half; c < half + 128; c += 32) {
              if (tn * BN + c >= p.N) break;
              uint32_t r[32];
              tmem_ld_32x32(taddr + c, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 o;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  o2[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]) * p.alpha,
                                                __uint_as_float(r[8 * j + 2 * e + 1]) * p.alpha);
                const int chunk = ((c - half) >> 3) + j;
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
              }
            }
            __syncwarp();
            const int chunks_valid = min(128, p.N - col_h) >> 3;
            const int ch = lane & 15;
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
              const int rr = 2 * i + (lane >> 4);
              if (quad * 32 + rr < rows && ch < chunks_valid) {
                const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((ch ^ (rr & 15)) << 4));
                const size_t orow = static_cast<size_t>(row0 + quad * 32 + rr - d_row_shift);
                *reinterpret_cast<uint4*>(dmat + orow * p.ldd + col_h + ch * 8) = v;
              }
            }
            __syncwarp();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        const int col = tn * BN + c;
        if (col >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        if (row_ok) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.N) v[i] += p.bias[col + i];
          }
          if (p.d_fp32) {
            float* dptr = reinterpret_cast<float*>(d_base) + row * p.ldd + col;
            const float* cptr = (GROUPED == 2 ? reinterpret_cast<const float*>(d_base) : reinterpret_cast<const float*>(p.C)) + row * p.ldc + col;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (col + i < p.N) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (p.beta != 0.f) {
                  const float4 cc = *reinterpret_cast<const float4*>(cptr + i);
                  o.x += p.beta * cc.x; o.y += p.beta * cc.y; o.z += p.beta * cc.z; o.w += p.beta * cc.w;
                }
                *reinterpret_cast<float4*>(dptr + i) = o;
              }
            }
          } else {
            __nv_bfloat16* dptr = reinterpret_cast<__nv_bfloat16*>(d_base) + row * p.ldd + col;
            const __nv_bfloat16* cptr = (GROUPED == 2 ? reinterpret_cast<const __nv_bfloat16*>(d_base) : reinterpret_cast<const __nv_bfloat16*>(p.C)) + row * p.ldc + col;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col + i < p.N) {
                if (p.beta != 0.f) {
                  const uint4 cc = *reinterpret_cast<const uint4*>(cptr + i);
                  const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&cc);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(c2[j]);
                    v[i + 2 * j] += p.beta * f.x;
                    v[i + 2 * j + 1] += p.beta * f.y;
                  }
                }
                uint4 o;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                *reinterpret_cast<uint4*>(dptr + i) = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
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

// Tensor map over a row-major bf16 tensor (dims innermost-first). box = {box0, box1[, 1]}.
// A training step launches the same few hundred (buffer, shape, tile) combinations tens of thousands of times (ring
// slots and weight views recur every round), so encoded maps are kept in a small direct-mapped table keyed on
// everything the encoding depends on: base address, extents, strides, box.  A map holds no data, only that
// description, so an entry stays valid when the memory behind the address is freed and reused.  (The reference's
// dispatcher keeps an exact-shape cache of its cuBLASLt plans for the same reason, helpers/matmul_dispatcher/src/
// dispatch.cpp:23-57.)
struct TmapKey {
  const void* base;
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  int rank;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rank == o.rank && dims[0] == o.dims[0] && dims[1] == o.dims[1] && dims[2] == o.dims[2] &&
           strides[0] == o.strides[0] && strides[1] == o.strides[1] && box[0] == o.box[0] && box[1] == o.box[1] &&
           box[2] == o.box[2];
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used = false;
};
constexpr int TMAP_SLOTS = 4096;
static int g_tmap_cache_on = 1;
static unsigned long long g_tmap_hits = 0, g_tmap_misses = 0;

static int make_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box) {
  static thread_local TmapSlot* table = nullptr;
  TmapKey key{};
  key.base = base; key.rank = rank;
  for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i < rank - 1; ++i) key.strides[i] = strides_bytes[i];
  TmapSlot* slot = nullptr;
  if (g_tmap_cache_on) {
    if (table == nullptr) table = new TmapSlot[TMAP_SLOTS];
    uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
    h ^= (key.dims[0] * 0xC2B2AE3D27D4EB4Full) ^ (key.dims[1] * 0x165667B19E3779F9ull) ^ (key.strides[0] << 7) ^
         (static_cast<uint64_t>(key.box[0]) << 40) ^ (static_cast<uint64_t>(key.box[1]) << 20) ^ key.dims[2];
    slot = &table[(h >> 24) & (TMAP_SLOTS - 1)];
    if (slot->used && slot->key == key) {
      *out = slot->map;
      ++g_tmap_hits;
      return 0;
    }
  }
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -100;
  cuuint64_t gdim[3];
  cuuint64_t gstr[2];
  cuuint32_t bx[3];
  cuuint32_t es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; }
  for (int i = 0; i < rank - 1; ++i) gstr[i] = strides_bytes[i];
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim, gstr, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -200 - static_cast<int>(r);
  ++g_tmap_misses;
  if (slot != nullptr) { slot->key = key; slot->map = *out; slot->used = true; }
  return 0;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int GROUPED, int COMM = 0>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_kernel<BN, STAGES, A_MN, B_MN, GROUPED, COMM>;
  constexpr int SMEM = L::TOTAL + (COMM == 2 ? RS_STAGE_BYTES : 0) + (COMM == 1 ? 2 * PULL_CHUNK_BYTES : 0);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return -300 - static_cast<int>(e);
    configured = true;
  }
  kern<<<grid, NUM_THREADS, SMEM, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - static_cast<int>(e);
}


// =====================================================================================================
// Two-SM variant (tcgen05 cta_group::2): a cluster of two CTAs owns one 256 x 256 output tile.  Each CTA stages its
// own 128 rows of A and HALF of the B tile (128 of the 256 N rows), so per 64-wide K block a CTA moves 32 KB instead
// of 48 KB for twice the math per pair: a third less L2 -> SM and shared-memory traffic, which is what bounds the
// one-SM kernel.  The leader CTA issues the MMAs for the pair; completion is multicast to both CTAs' barriers
// (tcgen05.commit); loads are plain tiled TMA loads credited to the leader's barrier (no cluster multicast loads).
// =====================================================================================================
constexpr int BN2 = 256;
constexpr int ST2 = 6;
constexpr int STAGE2_BYTES = 2 * BM * BK * 2;   // A (128 x 64) + B half (128 x 64)
constexpr int SMEM2_TOTAL = ST2 * STAGE2_BYTES + 256 + 1024;

// act(g) and d act / d g of the gate activation (same formulas as the stand-alone SwiGLU / GeGLU kernels)
__device__ __forceinline__ void glu_act_grad(float g, int kind, float& a, float& da) {
  if (kind == 0) {
    const float sg = 1.f / (1.f + __expf(-g));
    a = g * sg;
    da = sg * (1.f + g * (1.f - sg));
  } else {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float t = tanhf(k0 * (g + k1 * g * g * g));
    a = 0.5f * g * (1.f + t);
    da = 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
  }
}

// EPI selects the epilogue:
//   0  D = alpha * acc + beta * C + bias
//   1  gated-FFN forward.  B is the stacked [W_gate ; W_up] (2F x K, K-major).  A tile is 256 rows x (128 gate + 128 up)
//      columns: CTA 0 of the pair stages the gate rows of B, CTA 1 the up rows F below them, so the pair's accumulator
//      holds gate in columns 0..127 and up in 128..255.  The epilogue stores both halves into D (M x 2F, kept for the
//      backward) and act = act_fn(gate) * up into glu_act (M x F): the separate activation pass and its re-read of
//      the projection disappear (flextrain/ops/_kernels/swiglu.py:9-45 is that pass in the reference).
//   2  gated-FFN backward.  The accumulator is dact = dy · W_down; the epilogue reads the saved gate / up values and
//      writes dgate, dup into D (M x 2F) and the re-emitted activation into glu_act; dact never reaches memory
//      (flextrain/ops/_kernels/swiglu.py:46-100 reads it back from HBM).
template <bool A_MN, bool B_MN, int EPI = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + ST2 * STAGE2_BYTES);
  uint64_t* empty_bar = full_bar + ST2;
  uint64_t* tfull_bar = empty_bar + ST2;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = EPI == 1 ? p.glu_F / (BN2 / 2) : (p.N + BN2 - 1) / BN2;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < ST2; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 8); }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_slot, 512);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int row0 = tm * 2 * BM + static_cast<int>(cta) * BM;      // this CTA's 128 rows of A
        // this CTA's half of B's N rows (gated forward: 128 gate rows for CTA 0, the matching up rows for CTA 1)
        const int col0 = EPI == 1 ? tn * (BN2 / 2) + static_cast<int>(cta) * p.glu_F
                                  : tn * BN2 + static_cast<int>(cta) * (BN2 / 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, 50))) break;
          uint8_t* sa = smem + stage * STAGE2_BYTES;
          uint8_t* sb = sa + BM * BK * 2;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE2_BYTES);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d_2cta(sa, &tmA, &full_bar[stage], k0, row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_2cta(sa + j * (64 * BK * 2), &tmA, &full_bar[stage], row0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_2cta(sb, &tmB, &full_bar[stage], k0, col0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_2cta(sb + j * (64 * BK * 2), &tmB, &full_bar[stage], col0 + j * 64, k0);
          }
          if (++stage == ST2) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN2, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        if (!(ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, 60))) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN2;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(&full_bar[stage], phase, abort_flag, 61))) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE2_BYTES);
          const uint32_t sb = sa + BM * BK * 2;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_f16_2cta(tmem_d, ad, bd, idesc, (kb | kk) != 0);
          }
          umma_commit_2cta(&empty_bar[stage], 3);   // frees this stage in both CTAs
          if (++stage == ST2) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_2cta(&tfull_bar[acc], 3);       // accumulator ready in both CTAs
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int row0 = tm * 2 * BM + static_cast<int>(cta) * BM;
      const int rows = min(BM, p.M - row0);
      const int r_in = quad * 32 + lane;
      const bool row_ok = r_in < rows;
      const size_t row = static_cast<size_t>(row0 + r_in);
      // gated-FFN backward: saved gate / up values of 32 columns, fetched one step ahead of their use (the first
      // step is issued before the wait for the accumulator, it does not depend on the MMAs)
      [[maybe_unused]] uint4 xg[4], xu[4];
      [[maybe_unused]] auto fetch_x13 = [&](int col) {
        const __nv_bfloat16* xrow = reinterpret_cast<const __nv_bfloat16*>(p.glu_x13) + row * p.glu_ld_x13;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (row_ok && col + 8 * q < p.N) {
            xg[q] = __ldg(reinterpret_cast<const uint4*>(xrow + col + 8 * q));
            xu[q] = __ldg(reinterpret_cast<const uint4*>(xrow + p.glu_F + col + 8 * q));
          }
        }
      };
      if constexpr (EPI == 2) fetch_x13(tn * BN2);
      if (!(ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, 70))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN2;
      if constexpr (EPI == 1) {
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + row * p.ldd;
        __nv_bfloat16* arow = reinterpret_cast<__nv_bfloat16*>(p.glu_act) + row * p.glu_ld_act;
#pragma unroll 1
        for (int c = 0; c < BN2 / 2; c += 32) {
          const int col = tn * (BN2 / 2) + c;
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c, rg);
          tmem_ld_32x32(taddr + BN2 / 2 + c, ru);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 og, ou, oa;
              __nv_bfloat162* g2 = reinterpret_cast<__nv_bfloat162*>(&og);
              __nv_bfloat162* u2 = reinterpret_cast<__nv_bfloat162*>(&ou);
              __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&oa);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                g2[j] = __floats2bfloat162_rn(__uint_as_float(rg[i + 2 * j]), __uint_as_float(rg[i + 2 * j + 1]));
                u2[j] = __floats2bfloat162_rn(__uint_as_float(ru[i + 2 * j]), __uint_as_float(ru[i + 2 * j + 1]));
                // the activation is taken from the ROUNDED gate / up, exactly what the backward will read back
                const float2 gf = __bfloat1622float2(g2[j]), uf = __bfloat1622float2(u2[j]);
                float a0, a1, d0, d1;
                glu_act_grad(gf.x, p.glu_kind, a0, d0);
                glu_act_grad(gf.y, p.glu_kind, a1, d1);
                a2[j] = __floats2bfloat162_rn(a0 * uf.x, a1 * uf.y);
              }
              *reinterpret_cast<uint4*>(drow + col + i) = og;
              *reinterpret_cast<uint4*>(drow + p.glu_F + col + i) = ou;
              *reinterpret_cast<uint4*>(arow + col + i) = oa;
            }
          }
        }
      }
      if constexpr (EPI == 2) {
        __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(p.D) + row * p.ldd;
        __nv_bfloat16* arow = reinterpret_cast<__nv_bfloat16*>(p.glu_act) + row * p.glu_ld_act;
#pragma unroll 1
        for (int c = 0; c < BN2; c += 32) {
          const int col = tn * BN2 + c;
          if (col >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          uint4 cg[4], cu[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) { cg[q] = xg[q]; cu[q] = xu[q]; }
          if (c + 32 < BN2 && col + 32 < p.N) fetch_x13(col + 32);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int i = 8 * q;
              if (col + i < p.N) {
                const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&cg[q]);
                const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&cu[q]);
                uint4 odg, odu, oa;
                __nv_bfloat162* dg2 = reinterpret_cast<__nv_bfloat162*>(&odg);
                __nv_bfloat162* du2 = reinterpret_cast<__nv_bfloat162*>(&odu);
                __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&oa);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 gf = __bfloat1622float2(g2[j]), uf = __bfloat1622float2(u2[j]);
                  const float da0 = __uint_as_float(r[i + 2 * j]) * p.alpha, da1 = __uint_as_float(r[i + 2 * j + 1]) * p.alpha;
                  float a0, a1, d0, d1;
                  glu_act_grad(gf.x, p.glu_kind, a0, d0);
                  glu_act_grad(gf.y, p.glu_kind, a1, d1);
                  a2[j] = __floats2bfloat162_rn(a0 * uf.x, a1 * uf.y);
                  dg2[j] = __floats2bfloat162_rn(da0 * uf.x * d0, da1 * uf.y * d1);
                  du2[j] = __floats2bfloat162_rn(da0 * a0, da1 * a1);
                }
                *reinterpret_cast<uint4*>(drow + col + i) = odg;
                *reinterpret_cast<uint4*>(drow + p.glu_F + col + i) = odu;
                *reinterpret_cast<uint4*>(arow + col + i) = oa;
              }
            }
          }
        }
      }
      if constexpr (EPI == 0) {
#pragma unroll 1
      for (int c = 0; c < BN2; c += 32) {
        const int col = tn * BN2 + c;
        if (col >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        if (row_ok) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.N) v[i] += p.bias[col + i];
          }
          if (p.d_fp32) {
            float* dptr = reinterpret_cast<float*>(p.D) + row * p.ldd + col;
            const float* cptr = reinterpret_cast<const float*>(p.C) + row * p.ldc + col;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (col + i < p.N) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (p.beta != 0.f) {
                  const float4 cc = *reinterpret_cast<const float4*>(cptr + i);
                  o.x += p.beta * cc.x; o.y += p.beta * cc.y; o.z += p.beta * cc.z; o.w += p.beta * cc.w;
                }
                *reinterpret_cast<float4*>(dptr + i) = o;
              }
            }
          } else {
            __nv_bfloat16* dptr = reinterpret_cast<__nv_bfloat16*>(p.D) + row * p.ldd + col;
            const __nv_bfloat16* cptr = reinterpret_cast<const __nv_bfloat16*>(p.C) + row * p.ldc + col;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col + i < p.N) {
                if (p.beta != 0.f) {
                  const uint4 cc = *reinterpret_cast<const uint4*>(cptr + i);
                  const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&cc);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(c2[j]);
                    v[i + 2 * j] += p.beta * f.x;
                    v[i + 2 * j + 1] += p.beta * f.y;
                  }
                }
                uint4 o;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                *reinterpret_cast<uint4*>(dptr + i) = o;
              }
            }
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty_bar[acc]);   // 4 warps x 2 CTAs release the accumulator
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // the leader's MMAs also write the peer's TMEM: nobody frees before both are done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN, int EPI = 0>
static int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm2_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_TOTAL);
    if (e != cudaSuccess) return -300 - static_cast<int>(e);
    configured = true;
  }
  kern<<<grid, 192, SMEM2_TOTAL, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - static_cast<int>(e);
}

// D[m, n] = sum_s ws[s][m, n] + beta * C[m, n] + bias[n], four columns per thread (N % 8 == 0).
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, void* __restrict__ D,
                                     const void* __restrict__ C, const float* __restrict__ bias, int M, int N, int ldd,
                                     int ldc, float beta, int d_fp32) {
  const long i4 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long total4 = (long)M * N / 4;
  if (i4 >= total4) return;
  const long e = i4 * 4;
  const int m = (int)(e / N), n = (int)(e - (long)m * N);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sl = 0; sl < splits; ++sl) {
    const float4 v = *reinterpret_cast<const float4*>(ws + (size_t)sl * M * N + e);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  if (bias != nullptr) { acc.x += bias[n]; acc.y += bias[n + 1]; acc.z += bias[n + 2]; acc.w += bias[n + 3]; }
  if (d_fp32) {
    if (beta != 0.f) {
      const float4 c = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(C) + (size_t)m * ldc + n);
      acc.x += beta * c.x; acc.y += beta * c.y; acc.z += beta * c.z; acc.w += beta * c.w;
    }
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(D) + (size_t)m * ldd + n) = acc;
  } else {
    if (beta != 0.f) {
      const uint2 c = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(C) + (size_t)m * ldc + n);
      const float2 c0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&c.x));
      const float2 c1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&c.y));
      acc.x += beta * c0.x; acc.y += beta * c0.y; acc.z += beta * c1.x; acc.w += beta * c1.y;
    }
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(acc.x, acc.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(acc.z, acc.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(D) + (size_t)m * ldd + n) = o;
  }
}

template <int BN, int STAGES, int GROUPED>
static int dispatch_major(int a_mn, int b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                          int grid, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch<BN, STAGES, false, false, GROUPED>(ta, tb, p, grid, s);
  if (!a_mn && b_mn) return launch<BN, STAGES, false, true, GROUPED>(ta, tb, p, grid, s);
  if (a_mn && !b_mn) return launch<BN, STAGES, true, false, GROUPED>(ta, tb, p, grid, s);
  return launch<BN, STAGES, true, true, GROUPED>(ta, tb, p, grid, s);
}

}  // namespace ftb

using namespace ftb;

static int g_tp_pull_threads = 0;
static int g_use_2cta = 1;    // ftb_gemm_set_two_sm(0) falls back to the one-SM kernel for every shape
static int g_sm_count = 0;
static int sm_count() {
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sm_count;
}

extern "C" {

// D = alpha*op(A)*op(B) + beta*C + bias.   A, B bf16.  D/C bf16 (d_fp32=0) or fp32 (d_fp32=1).
//   a_mn_major = 0: A stored (M, K) row-major, leading dim lda;  1: A stored (K, M), leading dim lda.
//   b_mn_major = 0: B stored (N, K) row-major, leading dim ldb;  1: B stored (K, N), leading dim ldb.
// Requirements: base pointers 16-byte aligned, lda/ldb multiples of 8, ldd/ldc multiples of 8 (bf16) or 4 (fp32),
// N a multiple of 8.  Returns 0 or a negative error code.
int ftb_gemm_bf16(const void* A, const void* B, void* D, const void* C, const float* bias, int M, int N, int K,
                  int a_mn_major, int b_mn_major, int lda, int ldb, int ldd, int ldc, float alpha, float beta,
                  int d_fp32, int bn, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -1;
  if ((lda & 7) || (ldb & 7) || (N & 7) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(D) & 15))
    return -2;
  // bn == 512 selects the two-SM kernel (256 x 256 tile per CTA pair); bn == 0 picks it for large problems
  const bool two_sm = (bn == 512) || (bn == 0 && g_use_2cta && M >= 512 && N >= 512);
  if (two_sm) {
    CUtensorMap ta2, tb2;
    int rc2;
    if (!a_mn_major) {
      uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
      uint64_t str[1] = {(uint64_t)lda * 2};
      uint32_t box[2] = {BK, BM};
      rc2 = make_tmap(&ta2, A, 2, dims, str, box);
    } else {
      uint64_t dims[2] = {(uint64_t)M, (uint64_t)K};
      uint64_t str[1] = {(uint64_t)lda * 2};
      uint32_t box[2] = {64, BK};
      rc2 = make_tmap(&ta2, A, 2, dims, str, box);
    }
    if (rc2) return rc2;
    if (!b_mn_major) {
      uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
      uint64_t str[1] = {(uint64_t)ldb * 2};
      uint32_t box[2] = {BK, BM};                      // half of the 256-wide B tile per CTA
      rc2 = make_tmap(&tb2, B, 2, dims, str, box);
    } else {
      uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
      uint64_t str[1] = {(uint64_t)ldb * 2};
      uint32_t box[2] = {64, BK};
      rc2 = make_tmap(&tb2, B, 2, dims, str, box);
    }
    if (rc2) return rc2;
    GemmParams p2;
    p2.M = M; p2.N = N; p2.K = K; p2.ldd = ldd; p2.ldc = (C != nullptr) ? ldc : ldd;
    p2.alpha = alpha; p2.beta = (C != nullptr) ? beta : 0.f;
    p2.D = D; p2.C = (C != nullptr) ? C : D; p2.bias = bias; p2.d_fp32 = d_fp32;
    p2.num_groups = 0; p2.offsets = nullptr; p2.max_tiles = 0;
    p2.comm_mode = 0; p2.world = 1; p2.rank = 0; p2.panel_rows = 0; p2.split_k = 1; p2.k_per_split = 0;
    const int tiles2 = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN2 - 1) / BN2);
    int grid2 = sm_count() & ~1;
    if (max_ctas > 0 && max_ctas < grid2) grid2 = max_ctas & ~1;
    if (2 * tiles2 < grid2) grid2 = 2 * tiles2;
    if (grid2 < 2) grid2 = 2;
    if (!a_mn_major && !b_mn_major) return launch2<false, false>(ta2, tb2, p2, grid2, stream);
    if (!a_mn_major && b_mn_major) return launch2<false, true>(ta2, tb2, p2, grid2, stream);
    if (a_mn_major && !b_mn_major) return launch2<true, false>(ta2, tb2, p2, grid2, stream);
    return launch2<true, true>(ta2, tb2, p2, grid2, stream);
  }
  if (bn != 128 && bn != 256) bn = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn_major) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&ta, A, 2, dims, str, box);
  } else {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&ta, A, 2, dims, str, box);
  }
  if (rc) return rc;
  if (!b_mn_major) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {BK, (uint32_t)bn};
    rc = make_tmap(&tb, B, 2, dims, str, box);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&tb, B, 2, dims, str, box);
  }
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldc = (C != nullptr) ? ldc : ldd;
  p.alpha = alpha; p.beta = (C != nullptr) ? beta : 0.f;
  p.D = D; p.C = (C != nullptr) ? C : D; p.bias = bias; p.d_fp32 = d_fp32;
  p.num_groups = 0; p.offsets = nullptr; p.max_tiles = 0;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.panel_rows = 0; p.split_k = 1; p.k_per_split = 0;
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  if (bn == 256) return dispatch_major<256, 4, 0>(a_mn_major, b_mn_major, ta, tb, p, grid, stream);
  return dispatch_major<128, 6, 0>(a_mn_major, b_mn_major, ta, tb, p, grid, stream);
}

void ftb_gemm_set_two_sm(int on) { g_use_2cta = on; }
// tensor-map cache: switch, and (hits, misses) since the library was loaded
void ftb_gemm_set_tmap_cache(int on) { g_tmap_cache_on = on; }
void ftb_gemm_tmap_cache_stats(unsigned long long* hits, unsigned long long* misses) {
  *hits = g_tmap_hits; *misses = g_tmap_misses;
}
// all-gather -> GEMM: 1 = remote panels pulled by two warps of 16-byte loads, 0 (default) = by bulk copies
void ftb_gemm_set_tp_pull_threads(int on) { g_tp_pull_threads = on; }

// Gated-FFN forward in one kernel (two-SM tiles):  [gate | up] = X (M, K) @ W13 (2F, K)^T  ->  x13 (M, 2F), and
// act = act_fn(gate) * up -> act (M, F).  F must be a multiple of 128; X row-major with leading dimension lda,
// W13 contiguous rows (ldb), x13 leading dimension ld13, act leading dimension ld_act; kind 0 SwiGLU, 1 GeGLU(tanh).
int ftb_gemm_glu_fwd(const void* X, const void* W13, void* x13, void* act, int M, int F, int K, int lda, int ldb,
                     int ld13, int ld_act, int kind, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  if (K <= 0) return -1;
  if ((F % 128) || (lda & 7) || (ldb & 7) || (ld13 & 7) || (ld_act & 7) || (reinterpret_cast<uintptr_t>(X) & 15) ||
      (reinterpret_cast<uintptr_t>(W13) & 15) || (reinterpret_cast<uintptr_t>(x13) & 15) ||
      (reinterpret_cast<uintptr_t>(act) & 15))
    return -2;
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&ta, X, 2, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)(2 * F)};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&tb, W13, 2, dims, str, box);
    if (rc) return rc;
  }
  GemmParams p;
  p.M = M; p.N = 2 * F; p.K = K; p.ldd = ld13; p.ldc = ld13; p.alpha = 1.f; p.beta = 0.f;
  p.D = x13; p.C = x13; p.bias = nullptr; p.d_fp32 = 0;
  p.num_groups = 0; p.offsets = nullptr; p.max_tiles = 0;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.panel_rows = 0; p.split_k = 1; p.k_per_split = 0;
  p.glu_F = F; p.glu_kind = kind; p.glu_act = act; p.glu_ld_act = ld_act; p.glu_x13 = nullptr; p.glu_ld_x13 = 0;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * (F / 128);
  int grid = sm_count() & ~1;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas & ~1;
  if (2 * tiles < grid) grid = 2 * tiles;
  if (grid < 2) grid = 2;
  return launch2<false, false, 1>(ta, tb, p, grid, stream);
}

// Gated-FFN backward in one kernel:  dact = dY (M, K) @ W2 (K, F)  (never stored);  from the saved x13 = [gate | up]
// the epilogue writes dx13 = [dgate | dup] (M, 2F) and the re-emitted activation act (M, F).  F a multiple of 8.
int ftb_gemm_glu_bwd(const void* dY, const void* W2, const void* x13, void* dx13, void* act, int M, int F, int K,
                     int lda, int ldb, int ld13, int ldd13, int ld_act, int kind, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  if (K <= 0) return -1;
  if ((F & 7) || (lda & 7) || (ldb & 7) || (ld13 & 7) || (ldd13 & 7) || (ld_act & 7) ||
      (reinterpret_cast<uintptr_t>(dY) & 15) || (reinterpret_cast<uintptr_t>(W2) & 15) ||
      (reinterpret_cast<uintptr_t>(x13) & 15) || (reinterpret_cast<uintptr_t>(dx13) & 15) ||
      (reinterpret_cast<uintptr_t>(act) & 15))
    return -2;
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&ta, dY, 2, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)F, (uint64_t)K};       // W2 (K = d_model rows, F columns): MN-major B
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&tb, W2, 2, dims, str, box);
    if (rc) return rc;
  }
  GemmParams p;
  p.M = M; p.N = F; p.K = K; p.ldd = ldd13; p.ldc = ldd13; p.alpha = 1.f; p.beta = 0.f;
  p.D = dx13; p.C = dx13; p.bias = nullptr; p.d_fp32 = 0;
  p.num_groups = 0; p.offsets = nullptr; p.max_tiles = 0;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.panel_rows = 0; p.split_k = 1; p.k_per_split = 0;
  p.glu_F = F; p.glu_kind = kind; p.glu_act = act; p.glu_ld_act = ld_act; p.glu_x13 = x13; p.glu_ld_x13 = ld13;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((F + BN2 - 1) / BN2);
  int grid = sm_count() & ~1;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas & ~1;
  if (2 * tiles < grid) grid = 2 * tiles;
  if (grid < 2) grid = 2;
  return launch2<false, true, 2>(ta, tb, p, grid, stream);
}

// Split-K variant for small outputs with a long reduction (the rank-r LoRA gradients: M or N = r, K = tokens): the K
// range is cut into `splits` slices so that tiles x splits work items fill the GPU instead of a handful of CTAs each
// walking the whole K.  Every slice writes alpha * partial into its own fp32 slab of `workspace` (splits x M x N
// floats, supplied by the caller) and a second kernel adds the slabs (+ beta * C + bias) into D in the output type:
// fixed summation order, no atomics.  Same operand rules as ftb_gemm_bf16; one-SM kernel only.
int ftb_gemm_bf16_splitk(const void* A, const void* B, void* D, const void* C, const float* bias, int M, int N, int K,
                         int a_mn_major, int b_mn_major, int lda, int ldb, int ldd, int ldc, float alpha, float beta,
                         int d_fp32, int splits, float* workspace, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || splits < 2 || workspace == nullptr) return -1;
  if ((lda & 7) || (ldb & 7) || (N & 7) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(D) & 15))
    return -2;
  const int bn = (N <= 128) ? 128 : 256;
  int kps = ((K + splits - 1) / splits + BK - 1) / BK * BK;
  splits = (K + kps - 1) / kps;
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn_major) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&ta, A, 2, dims, str, box);
  } else {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&ta, A, 2, dims, str, box);
  }
  if (rc) return rc;
  if (!b_mn_major) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {BK, (uint32_t)bn};
    rc = make_tmap(&tb, B, 2, dims, str, box);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&tb, B, 2, dims, str, box);
  }
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldd = N; p.ldc = N;
  p.alpha = alpha; p.beta = 0.f;
  p.D = workspace; p.C = workspace; p.bias = nullptr; p.d_fp32 = 1;
  p.num_groups = 0; p.offsets = nullptr; p.max_tiles = 0;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.panel_rows = 0;
  p.split_k = splits; p.k_per_split = kps;
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn) * splits;
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  rc = (bn == 256) ? dispatch_major<256, 4, 0>(a_mn_major, b_mn_major, ta, tb, p, grid, stream)
                   : dispatch_major<128, 6, 0>(a_mn_major, b_mn_major, ta, tb, p, grid, stream);
  if (rc) return rc;
  const long n4 = (long)M * N / 4;
  splitk_reduce_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(workspace, splits, D, C != nullptr ? C : D,
                                                                         bias, M, N, ldd, C != nullptr ? ldc : ldd,
                                                                         C != nullptr ? beta : 0.f, d_fp32);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - static_cast<int>(e);
}

// Grouped GEMM over expert-major rows:  D[rows_g, :] = alpha * A[rows_g, :] * op(B[g]) + beta * C[rows_g, :].
//   A (total_rows, K) row-major; B (G, N, K) if b_mn_major = 0, (G, K, N) if 1; offsets (G+1) int32 on device.
//   max_tiles >= sum_g ceil(rows_g/128) * ceil(N/bn); the bound total_rows/128 + G row tiles always suffices.
int ftb_grouped_gemm_bf16(const void* A, const void* B, void* D, const void* C, const int* offsets, int num_groups,
                          int total_rows, int N, int K, int b_mn_major, int lda, int ldd, float alpha, float beta,
                          int d_fp32, int max_ctas, cudaStream_t stream) {
  if (total_rows <= 0 || N <= 0 || num_groups <= 0) return 0;
  if ((lda & 7) || (N & 7) || (K & 7)) return -2;
  const int bn = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)total_rows};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&ta, A, 2, dims, str, box);
    if (rc) return rc;
  }
  if (!b_mn_major) {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)num_groups};
    uint64_t str[2] = {(uint64_t)K * 2, (uint64_t)K * N * 2};
    uint32_t box[3] = {BK, (uint32_t)bn, 1};
    rc = make_tmap(&tb, B, 3, dims, str, box);
  } else {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)num_groups};
    uint64_t str[2] = {(uint64_t)N * 2, (uint64_t)K * N * 2};
    uint32_t box[3] = {64, BK, 1};
    rc = make_tmap(&tb, B, 3, dims, str, box);
  }
  if (rc) return rc;
  GemmParams p;
  p.M = total_rows; p.N = N; p.K = K; p.ldd = ldd; p.ldc = ldd;
  p.alpha = alpha; p.beta = (C != nullptr) ? beta : 0.f;
  p.D = D; p.C = (C != nullptr) ? C : D; p.bias = nullptr; p.d_fp32 = d_fp32;
  p.num_groups = num_groups; p.offsets = offsets;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.panel_rows = 0; p.split_k = 1; p.k_per_split = 0;
  const int tiles_n = (N + bn - 1) / bn;
  p.max_tiles = ((total_rows + BM - 1) / BM + num_groups) * tiles_n;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (p.max_tiles < grid) grid = p.max_tiles;
  if (bn == 256) return dispatch_major<256, 4, 1>(0, b_mn_major, ta, tb, p, grid, stream);
  return dispatch_major<128, 6, 1>(0, b_mn_major, ta, tb, p, grid, stream);
}

// Per-expert weight gradient in one launch:  G[g] (N, Kd) (+)= alpha * dY[rows_g, :N].T @ X[rows_g, :Kd]
//   dY (total_rows, N) and X (total_rows, Kd) row-major, expert-major rows, offsets (G+1) int32 on device; each expert's
//   row segment must start on a multiple of 64 and padding rows must be zero.  G is (num_groups, N, Kd) contiguous.
int ftb_grouped_wgrad_bf16(const void* dY, const void* X, void* G, const int* offsets, int num_groups, int total_rows,
                           int N, int Kd, int ldy, int ldx, float alpha, float beta, int g_fp32, int max_ctas,
                           cudaStream_t stream) {
  if (total_rows <= 0 || num_groups <= 0) return 0;
  if ((ldy & 7) || (ldx & 7) || (N & 7) || (Kd & 7)) return -2;
  const int bn = (Kd <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)total_rows};
    uint64_t str[1] = {(uint64_t)ldy * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&ta, dY, 2, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)Kd, (uint64_t)total_rows};
    uint64_t str[1] = {(uint64_t)ldx * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&tb, X, 2, dims, str, box);
    if (rc) return rc;
  }
  GemmParams p;
  p.M = N; p.N = Kd; p.K = total_rows; p.ldd = Kd; p.ldc = Kd; p.alpha = alpha; p.beta = beta;
  p.D = G; p.C = G; p.bias = nullptr; p.d_fp32 = g_fp32;
  p.num_groups = num_groups; p.offsets = offsets; p.max_tiles = 0;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.panel_rows = 0; p.split_k = 1; p.k_per_split = 0;
  const int tiles = num_groups * ((N + BM - 1) / BM) * ((Kd + bn - 1) / bn);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  if (bn == 256) return launch<256, 4, true, true, 2>(ta, tb, p, grid, stream);
  return launch<128, 6, true, true, 2>(ta, tb, p, grid, stream);
}

// Tensor-parallel fused GEMM.  A is (M, K) K-major with M = world * panel_rows.
//  mode 1 (all-gather -> GEMM): `a_local` is this rank's staging buffer of the full (M, K) matrix whose own panel
//    is already filled; `a_peer[r]` is rank r's staging buffer (same layout).  `panel_counter` (world x u64, device)
//    must be zero at launch.  D (M, N) is local.
//  mode 2 (GEMM -> reduce-scatter): A (M, K) is local; the partial output panel p is stored into
//    d_peer[p] + rank * d_slot_stride (elements) as a (panel_rows, N) matrix with leading dimension ldd.
// B as in ftb_gemm_bf16.  panel_rows must be a multiple of 128.
int ftb_gemm_bf16_tp(int mode, const void* A, void* const* a_peer, unsigned long long* panel_counter, const void* B,
                     void* D, void* const* d_peer, long d_slot_stride, int M, int N, int K, int b_mn_major, int lda,
                     int ldb, int ldd, float alpha, int d_fp32, int world, int rank, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || M % world) return -2;
  const int panel_rows = M / world;
  if (panel_rows % BM || (lda & 7) || (ldb & 7) || (N & 7)) return -2;
  const int bn = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&ta, A, 2, dims, str, box);
    if (rc) return rc;
  }
  if (!b_mn_major) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {BK, (uint32_t)bn};
    rc = make_tmap(&tb, B, 2, dims, str, box);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, BK};
    rc = make_tmap(&tb, B, 2, dims, str, box);
  }
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldc = ldd; p.alpha = alpha; p.beta = 0.f;
  p.D = D; p.C = D; p.bias = nullptr; p.d_fp32 = d_fp32;
  p.num_groups = 0; p.offsets = nullptr; p.max_tiles = 0;
  p.comm_mode = mode; p.world = world; p.rank = rank; p.panel_rows = panel_rows; p.split_k = 1; p.k_per_split = 0;
  p.pull_threads = g_tp_pull_threads;
  p.a_local = const_cast<void*>(A); p.panel_bytes = (long)panel_rows * lda * 2; p.panel_counter = panel_counter;
  p.d_slot_stride = d_slot_stride;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.a_peer[i] = (mode == 1 && i < world) ? a_peer[i] : nullptr;
    p.d_peer[i] = (mode == 2 && i < world) ? d_peer[i] : nullptr;
  }
  const int tiles = (M / BM) * ((N + bn - 1) / bn);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  if (mode == 1) {
    if (bn == 256) return b_mn_major ? launch<256, 4, false, true, 0, 1>(ta, tb, p, grid, stream)
                                     : launch<256, 4, false, false, 0, 1>(ta, tb, p, grid, stream);
    return b_mn_major ? launch<128, 6, false, true, 0, 1>(ta, tb, p, grid, stream)
                      : launch<128, 6, false, false, 0, 1>(ta, tb, p, grid, stream);
  }
  if (mode == 2) {
    if (bn == 256) return b_mn_major ? launch<256, 4, false, true, 0, 2>(ta, tb, p, grid, stream)
                                     : launch<256, 4, false, false, 0, 2>(ta, tb, p, grid, stream);
    return b_mn_major ? launch<128, 6, false, true, 0, 2>(ta, tb, p, grid, stream)
                      : launch<128, 6, false, false, 0, 2>(ta, tb, p, grid, stream);
  }
  return -2;
}

// Parameter all-gather fused into the first GEMM that consumes the gathered weights (comm mode 3).
//   D (M, N) = alpha * A (M, K) @ B (N, K)^T with B inside segment 0 of this rank's parameter arena `arena[rank]`.
//   Every segment s < nseg (byte offset seg_off[s], seg_numel[s] elements of seg_es[s] bytes) is sharded over the ranks
//   in element ranges of seg_per[s] elements; the kernel pulls the other ranks' ranges from `arena[r]` into the local
//   arena while it computes, so on return the whole layer is current.  `counters` (world x u64, device) must be zero.
//   Ranges must be multiples of 16 bytes.
int ftb_gemm_bf16_wgather(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldd, float alpha,
                          void* const* arena, int nseg, const long* seg_off, const long* seg_numel, const int* seg_es,
                          const long* seg_per, unsigned long long* counters, int world, int rank, int max_ctas,
                          cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || nseg < 1 || nseg > MAX_PULL) return -2;
  if ((lda & 7) || (N & 7) || (K & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  for (int s2 = 0; s2 < nseg; ++s2)
    if (((seg_per[s2] * seg_es[s2]) & 15) || ((seg_numel[s2] * seg_es[s2]) & 15) || (seg_off[s2] & 15)) return -2;
  const long gate_lo = static_cast<long>(reinterpret_cast<const char*>(B) - reinterpret_cast<const char*>(arena[rank])) -
                       seg_off[0];
  if (gate_lo < 0 || gate_lo + static_cast<long>(N) * K * 2 > seg_numel[0] * seg_es[0]) return -2;
  const int bn = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BK, BM};
    rc = make_tmap(&ta, A, 2, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)K * 2};
    uint32_t box[2] = {BK, (uint32_t)bn};
    rc = make_tmap(&tb, B, 2, dims, str, box);
    if (rc) return rc;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ldc = ldd; p.alpha = alpha; p.beta = 0.f;
  p.D = D; p.C = D; p.bias = nullptr; p.d_fp32 = 0;
  p.num_groups = 0; p.offsets = nullptr; p.max_tiles = 0;
  p.comm_mode = 3; p.world = world; p.rank = rank; p.panel_rows = 0; p.split_k = 1; p.k_per_split = 0;
  p.a_local = arena[rank]; p.panel_bytes = 0; p.panel_counter = counters; p.d_slot_stride = 0;
  for (int i = 0; i < MAX_RANKS; ++i) { p.a_peer[i] = i < world ? arena[i] : nullptr; p.d_peer[i] = nullptr; }
  p.n_pull = nseg;
  for (int s2 = 0; s2 < MAX_PULL; ++s2) {
    p.pull_off[s2] = s2 < nseg ? seg_off[s2] : 0; p.pull_numel[s2] = s2 < nseg ? seg_numel[s2] : 0;
    p.pull_per[s2] = s2 < nseg ? seg_per[s2] : 1; p.pull_es[s2] = s2 < nseg ? seg_es[s2] : 2;
  }
  p.gate_lo = gate_lo;
  const int tiles_n = (N + bn - 1) / bn;
  const long my_lo = min(seg_numel[0], rank * seg_per[0]) * seg_es[0];        // first byte of my range in segment 0
  long first = (my_lo - gate_lo) / (static_cast<long>(bn) * K * 2);
  if (my_lo <= gate_lo) first = 0;
  p.tn_first = static_cast<int>(first >= tiles_n ? 0 : first);
  const int tiles = ((M + BM - 1) / BM) * tiles_n;
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  if (bn == 256) return launch<256, 4, false, false, 0, 3>(ta, tb, p, grid, stream);
  return launch<128, 6, false, false, 0, 3>(ta, tb, p, grid, stream);
}

// Reads and clears the library's device error word: returns code * 1000 + where (0 = no error).
int ftb_gemm_error(void) {
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
