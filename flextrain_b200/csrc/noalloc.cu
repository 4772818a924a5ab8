// ftb_rmsnorm_bwd_noalloc: RMSNorm backward whose reduction workspace is a static device array.
// See noalloc.h for who needs this and for the full contract.
#include "noalloc.h"

#include <cuda_bf16.h>
#include <stdint.h>

namespace {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// The workspace.  In HOST code this name is only a stand-in for the symbol: it is not a device address, and
// handing it to a kernel would fault (or, where the GPU can reach host memory, quietly use the wrong memory).
// Host code therefore asks the runtime for the device address once per device (resolve_scratch below).
static __device__ __align__(256) float g_scratch[FTB_NOALLOC_MAX_BLOCKS * FTB_NOALLOC_MAX_D];

constexpr int THREADS = 256;
constexpr int MAXV = FTB_NOALLOC_MAX_D / (8 * THREADS);   // 16-byte vectors per thread per row
constexpr int MAX_DEVICES = 64;
static float* g_scratch_dev[MAX_DEVICES] = {nullptr};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? sh[l] : 0.f;
  return warp_sum(t);
}
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
__device__ __forceinline__ void load_w(const float* w, int i, float (&wf)[8]) {
  if (w) {
    const float4 a = reinterpret_cast<const float4*>(w)[2 * i];
    const float4 b = reinterpret_cast<const float4*>(w)[2 * i + 1];
    wf[0] = a.x; wf[1] = a.y; wf[2] = a.z; wf[3] = a.w; wf[4] = b.x; wf[5] = b.y; wf[6] = b.z; wf[7] = b.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) wf[e] = 1.f;
  }
}

// dx = (dy*w - xhat * mean(dy*w*xhat)) * rstd (+ dx_add); y_out = xhat * w; partial[block, :] = sum_rows dy * xhat.
// Every block writes its whole row of `partial` (zeros included), so stale workspace contents are never read.
__global__ void __launch_bounds__(THREADS) bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                      const float* __restrict__ w, const float* __restrict__ rstd,
                                                      const bf16* __restrict__ dx_add, bf16* __restrict__ dx,
                                                      bf16* __restrict__ y_out, float* __restrict__ partial, int T,
                                                      int D) {
  __shared__ float sh[32];
  const int nv = D >> 3;
  float acc[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * D);
    const float r = rstd[row];
    uint4 xv[MAXV], gv[MAXV];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nv) {
        xv[j] = xr[i];
        gv[j] = gr[i];
        float xf[8], gf[8], wf[8];
        unpack8(xv[j], xf);
        unpack8(gv[j], gf);
        load_w(w, i, wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = xf[e] * r;
          acc[j][e] += gf[e] * xh;
          dot += gf[e] * wf[e] * xh;
        }
      }
    }
    dot = block_sum(dot, sh) / (float)D;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nv) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xv[j], xf);
        unpack8(gv[j], gf);
        load_w(w, i, wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (gf[e] * wf[e] - xf[e] * r * dot) * r;
        if (dx_add) {
          float a[8];
          unpack8(reinterpret_cast<const uint4*>(dx_add + (size_t)row * D)[i], a);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += a[e];
        }
        reinterpret_cast<uint4*>(dx + (size_t)row * D)[i] = pack8(o);
        if (y_out) {
          float yv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) yv[e] = xf[e] * r * wf[e];
          reinterpret_cast<uint4*>(y_out + (size_t)row * D)[i] = pack8(yv);
        }
      }
    }
  }
  if (partial) {
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < nv) {
        float* o = partial + (size_t)blockIdx.x * D + i * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = acc[j][e];
      }
    }
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int P, int D, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[(size_t)p * D + c];
  out[c] = accumulate ? out[c] + s : s;
}

// Device address of g_scratch on the current device; resolved once per device, never allocates.  The cache is
// written without a lock: two host threads that race here both store the same address, which is harmless.
int resolve_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return FTB_NOALLOC_ERR_SYMBOL;
  if (g_scratch_dev[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess || p == nullptr) return FTB_NOALLOC_ERR_SYMBOL;
    g_scratch_dev[dev] = p;
  }
  *out = g_scratch_dev[dev];
  return 0;
}

}  // namespace

extern "C" {

int ftb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, const void* dx_add,
                            void* dx, void* y_out, float* dw, int dw_accumulate, int T, int D, cudaStream_t stream) {
  if (T < 0 || D <= 0 || (D & 7)) return FTB_NOALLOC_ERR_BAD_SHAPE;
  if (D > FTB_NOALLOC_MAX_D) return FTB_NOALLOC_ERR_TOO_LARGE;
  // Host-side pointer checks (nothing is launched on failure).  The kernels move rows as 16-byte vectors, so an
  // unaligned view of a caller's buffer would fault on the device; a weight gradient without weights has no meaning.
  if (dy == nullptr || x == nullptr || rstd == nullptr || dx == nullptr) return FTB_NOALLOC_ERR_BAD_POINTER;
  const void* vec_ptrs[] = {dy, x, dx, dx_add, y_out, w, dw};
  for (const void* q : vec_ptrs)
    if (q != nullptr && (reinterpret_cast<uintptr_t>(q) & 15)) return FTB_NOALLOC_ERR_BAD_POINTER;
  if ((reinterpret_cast<uintptr_t>(rstd) & 3)) return FTB_NOALLOC_ERR_BAD_POINTER;
  if (dw != nullptr && w == nullptr) return FTB_NOALLOC_ERR_BAD_POINTER;
  if (T == 0) return 0;
  float* scratch = nullptr;
  const int rc = resolve_scratch(&scratch);
  if (rc != 0) return rc;
  const int blocks = T < FTB_NOALLOC_MAX_BLOCKS ? T : FTB_NOALLOC_MAX_BLOCKS;
  const bool want_dw = (dw != nullptr) && (w != nullptr);
  bwd_kernel<<<blocks, THREADS, 0, stream>>>((const bf16*)dy, (const bf16*)x, w, rstd, (const bf16*)dx_add, (bf16*)dx,
                                             (bf16*)y_out, want_dw ? scratch : nullptr, T, D);
  if (want_dw) colsum_kernel<<<(D + 255) / 256, 256, 0, stream>>>(scratch, dw, blocks, D, dw_accumulate);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - (int)e;
}

const char* ftb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case FTB_NOALLOC_ERR_TOO_LARGE:
      return "row width D exceeds FTB_NOALLOC_MAX_D (8192): the built-in workspace cannot hold the reduction";
    case FTB_NOALLOC_ERR_BAD_SHAPE: return "D must be a positive multiple of 8 and T must not be negative";
    case FTB_NOALLOC_ERR_BAD_POINTER:
      return "dy, x, rstd, dx are required; every tensor pointer must be 16-byte aligned; dw needs w";
    case FTB_NOALLOC_ERR_SYMBOL: return "could not resolve the device address of the built-in workspace";
    default: return "CUDA launch error (code = -400 - cudaError_t)";
  }
}

}  // extern "C"
