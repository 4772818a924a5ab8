// Expert-parallel dispatch / combine over peer memory (one process per GPU, experts sharded over ranks).
//
// The reference runs every expert on one GPU behind a host sync (flextrain/ops/full_moe.py:134-148); there is no
// expert parallelism to port.  Here each rank routes its own tokens, and:
//
//   ftb_ep_push_rows     dispatch: every routed (token, k) slot's activation row is stored straight into the owning
//                        rank's expert-major receive buffer (peer stores; destination rows are computed on the
//                        device from the all-gathered per-(rank, expert) counts), optionally with a per-row scalar
//                        (the router weight, needed by the owner in backward).
//   ftb_ep_combine_pull  combine: out[t] = resid[t] + sum_k w[t,k] * Y_owner[row(t,k)] read from the owners' output
//                        buffers (peer loads) with fp32 accumulation — the weighted K-way gather of the reference
//                        (flextrain/ops/_kernels/moe.py:560-598) fused with the return all-to-all.
//   ftb_ep_pull_scalar   per-slot scalar read back from the owners (router-weight gradients).
//
// The grouped expert GEMMs between dispatch and combine are the tcgen05 grouped kernels of gemm_tcgen05.cu.
// Rows whose destination exceeds the receive capacity are skipped and recorded in the error word (3): capacity
// overflow is reported, never silently dropped or written out of bounds.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;
constexpr int MAX_RANKS = 8;

static __device__ int g_error_word = 0;
static __device__ int g_error_where = 0;
__device__ __forceinline__ void set_error(int code, int where) {
  if (atomicCAS(&g_error_word, 0, code) == 0) g_error_where = where;
}

struct PeerTable {
  void* ptr[MAX_RANKS];
};

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// One CTA per routed slot i (expert-sorted order): recv[dest_rank[i]][dest_row[i], :] = x[src_tok[i], :].
__global__ void ep_push_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ src_tok,
                                    const int* __restrict__ dest_rank, const int* __restrict__ dest_row,
                                    const float* __restrict__ scalar, PeerTable recv, PeerTable recv_scalar, long n,
                                    int D, long capacity) {
  const long i = blockIdx.x;
  if (i >= n) return;
  const int dr = dest_rank[i];
  const long row = dest_row[i];
  if (dr < 0) return;
  if (row >= capacity) {
    if (threadIdx.x == 0) set_error(3, dr);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)src_tok[i] * D);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(recv.ptr[dr]) + row * D);
  for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) dst[c] = src[c];
  if (scalar != nullptr && threadIdx.x == 0) reinterpret_cast<float*>(recv_scalar.ptr[dr])[row] = scalar[i];
}

// out[t, :] = resid[t, :] + sum_k w[t,k] * Y[rank(t,k)][row(t,k), :]
__global__ void ep_combine_pull_kernel(PeerTable ybufs, const int* __restrict__ slot_rank, const int* __restrict__ slot_row,
                                       const float* __restrict__ w, const bf16* __restrict__ resid, bf16* __restrict__ out,
                                       int T, int K, int D, long capacity) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (resid) unpack8(reinterpret_cast<const uint4*>(resid + (size_t)t * D)[c], acc);
    for (int k = 0; k < K; ++k) {
      const int r = slot_rank[(size_t)t * K + k];
      const long row = slot_row[(size_t)t * K + k];
      if (r < 0 || row >= capacity) continue;
      const float wk = w ? w[(size_t)t * K + k] : 1.f;
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(ybufs.ptr[r]) + row * D)[c], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += wk * f[e];
    }
    reinterpret_cast<uint4*>(out + (size_t)t * D)[c] = pack8(acc);
  }
}

__global__ void ep_pull_scalar_kernel(PeerTable sbufs, const int* __restrict__ slot_rank, const int* __restrict__ slot_row,
                                      float* __restrict__ out, long n, long capacity) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = slot_rank[i];
  const long row = slot_row[i];
  out[i] = (r < 0 || row >= capacity) ? 0.f : reinterpret_cast<const float*>(sbufs.ptr[r])[row];
}


// ------------------------------------------------------------------------------------------------------------
// Device-side routing plan: a stable counting sort of the T*K (token, k) slots by expert, with every expert's row
// segment padded to the GEMM tile height.  Three small launches, no host read, no atomics on global memory (the
// result is deterministic and equal to a stable sort):
//   hist   each block counts the experts of its PLAN_CHUNK consecutive slots (shared-memory histogram)
//   scan   one block turns the per-block counts into exclusive prefixes per expert, and the totals into offsets
//   map    each block walks its slots in order and gives slot i the row  offsets[e] + (slots of e before i)
// The reference does this with count / prefix-sum / map kernels followed by a copy of the counts to pinned host
// memory and a stream synchronize (flextrain/ops/_kernels/moe.py:318-357,461-505; flextrain/ops/full_moe.py:134-148).
// ------------------------------------------------------------------------------------------------------------
constexpr int PLAN_THREADS = 256;
constexpr int PLAN_WARPS = PLAN_THREADS / 32;
constexpr int PLAN_CHUNK = 2048;
constexpr int PLAN_MAX_E = 1024;

__global__ void moe_hist_kernel(const int* __restrict__ experts, long n, int E, int* __restrict__ bh,
                                int* __restrict__ fill, long fill_n) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const long lo = (long)blockIdx.x * PLAN_CHUNK;
  const long hi = min(n, lo + PLAN_CHUNK);
  for (long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const int e = experts[i];
    if ((unsigned)e < (unsigned)E) atomicAdd(&sh[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) bh[(long)blockIdx.x * E + e] = sh[e];
  // rows that no slot lands on (tile padding, the unused tail) read as "no source"
  if (fill != nullptr)
    for (long r = (long)blockIdx.x * blockDim.x + threadIdx.x; r < fill_n; r += (long)gridDim.x * blockDim.x) fill[r] = -1;
}

// bh (nb x E): counts -> exclusive prefix over blocks; counts[e] = total; offsets (E+1) = padded exclusive scan.
__global__ void moe_scan_kernel(int* __restrict__ bh, int nb, int E, int pad, int* __restrict__ counts,
                                int* __restrict__ offsets) {
  __shared__ int padded[PLAN_MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int b = 0; b < nb; ++b) {
      const int t = bh[(long)b * E + e];
      bh[(long)b * E + e] = run;
      run += t;
    }
    counts[e] = run;
    padded[e] = (run + pad - 1) / pad * pad;
  }
  __syncthreads();
  if (threadIdx.x == 0 && offsets != nullptr) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = acc;
      acc += padded[e];
    }
    offsets[E] = acc;
  }
}

// Expert parallel: from the all-gathered (W x E) count table, the first row of THIS rank's slots of expert e inside the
// owner's expert-major buffer (start[e]) and the padded row offsets of this rank's own experts (clamped to capacity).
__global__ void ep_scan_kernel(const int* __restrict__ table, int W, int E, int rank, int pad, long capacity,
                               int* __restrict__ start, int* __restrict__ my_offsets) {
  __shared__ int padded[PLAN_MAX_E];
  __shared__ int before[PLAN_MAX_E];
  const int El = E / W;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, bef = 0;
    for (int r = 0; r < W; ++r) {
      const int c = table[(long)r * E + e];
      if (r < rank) bef += c;
      tot += c;
    }
    padded[e] = (tot + pad - 1) / pad * pad;
    before[e] = bef;
  }
  __syncthreads();
  if (threadIdx.x < W) {
    const int o = threadIdx.x;
    long acc = 0;
    for (int j = 0; j < El; ++j) {
      const int e = o * El + j;
      start[e] = (int)(acc + before[e]);
      if (o == rank) my_offsets[j] = (int)min(acc, capacity);
      acc += padded[e];
    }
    if (o == rank) my_offsets[El] = (int)min(acc, capacity);
  }
}

// mode 0 (one GPU): inv[i] = row, row_src[row] = i.   mode 1 (expert parallel): slot_rank[i] = owner, slot_row[i] = row.
__global__ void moe_map_kernel(const int* __restrict__ experts, long n, int E, const int* __restrict__ bh,
                               const int* __restrict__ first_row, int* __restrict__ out_a, int* __restrict__ out_b,
                               int mode, int El, long capacity, int* __restrict__ overflow) {
  extern __shared__ int sh[];
  int* base = sh;            // [E]   next free row of expert e for this block
  int* wc = sh + E;          // [PLAN_WARPS][E]  slots of e seen by warp w in the current pass
  for (int e = threadIdx.x; e < E; e += blockDim.x) base[e] = first_row[e] + bh[(long)blockIdx.x * E + e];
  for (int j = threadIdx.x; j < PLAN_WARPS * E; j += blockDim.x) wc[j] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long lo = (long)blockIdx.x * PLAN_CHUNK;
  const long hi = min(n, lo + PLAN_CHUNK);
  for (long it = lo; it < hi; it += blockDim.x) {
    const long i = it + threadIdx.x;
    int e = i < hi ? experts[i] : -1;
    const bool valid = (unsigned)e < (unsigned)E;
    const unsigned m = __match_any_sync(0xffffffffu, valid ? e : -1 - lane);
    const int in_warp = __popc(m & ((1u << lane) - 1u));
    if (valid && in_warp == 0) wc[warp * E + e] = __popc(m);
    __syncthreads();
    if (valid) {
      int prefix = 0;
      for (int w2 = 0; w2 < warp; ++w2) prefix += wc[w2 * E + e];
      const long row = (long)base[e] + prefix + in_warp;
      if (mode == 0) {
        out_a[i] = (int)row;               // inv
        out_b[row] = (int)i;               // row_src
      } else {
        const int owner = e / El;
        out_a[i] = owner;                  // slot_rank
        out_b[i] = (int)row;               // slot_row
        if (row >= capacity && overflow != nullptr) *overflow = 1;
      }
    } else if (i < hi && mode == 1) {
      out_a[i] = -1;
      out_b[i] = 0;
    }
    __syncthreads();
    for (int e2 = threadIdx.x; e2 < E; e2 += blockDim.x) {
      int s2 = 0;
#pragma unroll
      for (int w2 = 0; w2 < PLAN_WARPS; ++w2) {
        s2 += wc[w2 * E + e2];
        wc[w2 * E + e2] = 0;
      }
      base[e2] += s2;
    }
    __syncthreads();
  }
}

// Dispatch by slot (token-major): warp per (token, k) slot, recv[slot_rank][slot_row, :] = x[slot / K, :].  The K slots
// of a token sit in one CTA, so the token's row is read from HBM once; every lane keeps eight 16-byte loads in flight
// before the (peer) stores.
__global__ void ep_push_slots_kernel(const bf16* __restrict__ x, const int* __restrict__ slot_rank,
                                     const int* __restrict__ slot_row, const float* __restrict__ scalar, PeerTable recv,
                                     PeerTable recv_scalar, long n, int K, int D, long capacity) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long slot = (long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (slot >= n) return;
  const int dr = slot_rank[slot];
  const long row = slot_row[slot];
  if (dr < 0) return;
  if (row >= capacity) {
    if (lane == 0) set_error(3, dr);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(slot / K) * D);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(recv.ptr[dr]) + row * D);
  const int nv = D >> 3;
  int c = lane;
  for (; c + 7 * 32 < nv; c += 8 * 32) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = src[c + u * 32];
#pragma unroll
    for (int u = 0; u < 8; ++u) dst[c + u * 32] = v[u];
  }
  for (; c < nv; c += 32) dst[c] = src[c];
  if (scalar != nullptr && lane == 0) reinterpret_cast<float*>(recv_scalar.ptr[dr])[row] = scalar[slot];
}

}  // namespace

#define CHECK_LAUNCH()                                 \
  do {                                                 \
    cudaError_t e_ = cudaGetLastError();               \
    return e_ == cudaSuccess ? 0 : -400 - (int)e_;     \
  } while (0)

static void fill(PeerTable& t, void* const* p, int world) {
  for (int i = 0; i < MAX_RANKS; ++i) t.ptr[i] = (p != nullptr && i < world) ? p[i] : nullptr;
}

extern "C" {

int ftb_ep_push_rows(const void* x, const int* src_tok, const int* dest_rank, const int* dest_row, const float* scalar,
                     void* const* recv, void* const* recv_scalar, long n, int D, long capacity, int world,
                     cudaStream_t s) {
  if (n == 0) return 0;
  if (world > MAX_RANKS || (D & 7)) return -2;
  PeerTable a, b;
  fill(a, recv, world);
  fill(b, recv_scalar, world);
  ep_push_rows_kernel<<<(unsigned)n, 128, 0, s>>>((const bf16*)x, src_tok, dest_rank, dest_row, scalar, a, b, n, D,
                                                  capacity);
  CHECK_LAUNCH();
}

// Routing plan on one GPU.  experts (n = T*K, int32), E <= 1024.  Outputs: counts (E), offsets (E+1, segments padded to
// `pad`), inv (n): row of every slot, row_src (R): slot of every row or -1.  work: ceil(n / 2048) * E ints of scratch.
// R must be at least n + E * (pad - 1) rounded up to `pad`.
int ftb_moe_plan(const int* experts, long n, int E, int pad, long R, int* work, int* counts, int* offsets, int* inv,
                 int* row_src, cudaStream_t s) {
  if (n <= 0) return 0;
  if (E <= 0 || E > PLAN_MAX_E || pad <= 0) return -2;
  const int nb = (int)((n + PLAN_CHUNK - 1) / PLAN_CHUNK);
  moe_hist_kernel<<<nb, PLAN_THREADS, E * sizeof(int), s>>>(experts, n, E, work, row_src, R);
  moe_scan_kernel<<<1, 1024, 0, s>>>(work, nb, E, pad, counts, offsets);
  moe_map_kernel<<<nb, PLAN_THREADS, (1 + PLAN_WARPS) * E * sizeof(int), s>>>(experts, n, E, work, offsets, inv, row_src,
                                                                               0, 1, 0, nullptr);
  CHECK_LAUNCH();
}

// Expert-parallel plan, first half: this rank's per-expert counts (to be all-gathered) and the per-block prefixes.
int ftb_ep_plan_count(const int* experts, long n, int E, int* work, int* counts, cudaStream_t s) {
  if (E <= 0 || E > PLAN_MAX_E) return -2;
  const int nb = (int)((n + PLAN_CHUNK - 1) / PLAN_CHUNK);
  if (nb == 0) return cudaMemsetAsync(counts, 0, E * sizeof(int), s) == cudaSuccess ? 0 : -400;
  moe_hist_kernel<<<nb, PLAN_THREADS, E * sizeof(int), s>>>(experts, n, E, work, nullptr, 0);
  moe_scan_kernel<<<1, 1024, 0, s>>>(work, nb, E, 1, counts, nullptr);
  CHECK_LAUNCH();
}

// Second half, after the (W x E) table of all ranks' counts is complete: destination rank and row of every slot
// (slot_rank, slot_row: n ints each), the padded row offsets of this rank's own experts (E/W + 1 ints, clamped to
// `capacity`), and *overflow = 1 if a destination row does not fit the capacity.  start: E ints of scratch.
int ftb_ep_plan_map(const int* experts, long n, int E, const int* table, int W, int rank, int pad, long capacity,
                    const int* work, int* start, int* my_offsets, int* slot_rank, int* slot_row, int* overflow,
                    cudaStream_t s) {
  if (E <= 0 || E > PLAN_MAX_E || W <= 0 || W > MAX_RANKS || E % W) return -2;
  ep_scan_kernel<<<1, 1024, 0, s>>>(table, W, E, rank, pad, capacity, start, my_offsets);
  const int nb = (int)((n + PLAN_CHUNK - 1) / PLAN_CHUNK);
  if (nb > 0)
    moe_map_kernel<<<nb, PLAN_THREADS, (1 + PLAN_WARPS) * E * sizeof(int), s>>>(experts, n, E, work, start, slot_rank,
                                                                                 slot_row, 1, E / W, capacity, overflow);
  CHECK_LAUNCH();
}

int ftb_ep_push_slots(const void* x, const int* slot_rank, const int* slot_row, const float* scalar, void* const* recv,
                      void* const* recv_scalar, long n, int K, int D, long capacity, int world, cudaStream_t s) {
  if (n == 0) return 0;
  if (world > MAX_RANKS || (D & 7) || K <= 0) return -2;
  PeerTable a, b;
  fill(a, recv, world);
  fill(b, recv_scalar, world);
  const int warps = 8;
  ep_push_slots_kernel<<<(unsigned)((n + warps - 1) / warps), warps * 32, 0, s>>>((const bf16*)x, slot_rank, slot_row, scalar,
                                                                                   a, b, n, K, D, capacity);
  CHECK_LAUNCH();
}

int ftb_ep_combine_pull(void* const* ybufs, const int* slot_rank, const int* slot_row, const float* w, const void* resid,
                        void* out, int T, int K, int D, long capacity, int world, cudaStream_t s) {
  if (T == 0) return 0;
  if (world > MAX_RANKS || (D & 7)) return -2;
  PeerTable a;
  fill(a, ybufs, world);
  ep_combine_pull_kernel<<<T, 128, 0, s>>>(a, slot_rank, slot_row, w, (const bf16*)resid, (bf16*)out, T, K, D, capacity);
  CHECK_LAUNCH();
}

int ftb_ep_pull_scalar(void* const* sbufs, const int* slot_rank, const int* slot_row, float* out, long n, long capacity,
                       int world, cudaStream_t s) {
  if (n == 0) return 0;
  if (world > MAX_RANKS) return -2;
  PeerTable a;
  fill(a, sbufs, world);
  ep_pull_scalar_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, slot_rank, slot_row, out, n, capacity);
  CHECK_LAUNCH();
}

int ftb_moe_error(void) {
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
