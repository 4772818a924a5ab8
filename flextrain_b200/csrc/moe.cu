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
