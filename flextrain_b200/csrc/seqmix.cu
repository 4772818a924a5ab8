// Element-wise / small-reduction kernels around the Gated DeltaNet recurrence (sm_100a): depthwise causal conv1d
// with SiLU and cross-chunk state (forward / backward), per-head L2 normalisation with a token stride (forward /
// backward), gated RMSNorm backward, and a top-p sampler.  The reference project takes these from FLA / Triton
// (flextrain/nn/blocks/linear_attn.py:168-255, 1806-1843; flextrain/ops/_kernels/l2norm.py:27-99,
// gated_rmsnorm.py:224-357, sample_top_p.py:7-150).  All are memory-bound: one pass over the data, fp32 math.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

typedef __nv_bfloat16 bf16;
constexpr int MAXW = 8;     // conv width limit

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// sequence index of token t: largest s with cu[s] <= t
__device__ __forceinline__ int seq_of(const int* __restrict__ cu, int nseq, int t) {
  int lo = 0, hi = nseq;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid;
  }
  return lo;
}

// "virtual input" of a sequence at position pos in [-(W-1), L): x for pos >= 0, the carried state before that
__device__ __forceinline__ float conv_input(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ init, int D,
                                            int W, int seq, int a, int pos, int d) {
  if (pos >= 0) return __bfloat162float(x[(long)(a + pos) * ldx + d]);
  if (init == nullptr) return 0.f;
  return __bfloat162float(init[((long)seq * D + d) * (W - 1) + (W - 1) + pos]);
}

// y[t, d] = act( sum_j w[d, j] * in(pos - (W-1) + j) ),  thread = channel, block row = TT tokens
template <int TT>
__global__ void conv1d_fwd_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ w,
                                  const bf16* __restrict__ init, const int* __restrict__ cu, int nseq, bf16* __restrict__ y,
                                  int T, int D, int W, int act) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float wr[MAXW];
  for (int j = 0; j < W; ++j) wr[j] = __bfloat162float(w[(long)d * W + j]);
  const int tb = blockIdx.y * TT;
  for (int t = tb; t < min(T, tb + TT); ++t) {
    const int s = seq_of(cu, nseq, t), a = cu[s], pos = t - a;
    float acc = 0.f;
    for (int j = 0; j < W; ++j) acc += wr[j] * conv_input(x, ldx, init, D, W, s, a, pos - (W - 1) + j, d);
    y[(long)t * D + d] = __float2bfloat16(act ? acc * sigmoidf(acc) : acc);
  }
}

// final_state[s, d, m] = virtual input at position L - (W-1) + m
__global__ void conv1d_state_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ init,
                                    const int* __restrict__ cu, bf16* __restrict__ fin, int D, int W) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (d >= D) return;
  const int a = cu[s], L = cu[s + 1] - a;
  for (int m = 0; m < W - 1; ++m) {
    const int pos = L - (W - 1) + m;
    float v = 0.f;
    if (pos >= -(W - 1)) v = conv_input(x, ldx, init, D, W, s, a, pos, d);
    fin[((long)s * D + d) * (W - 1) + m] = __float2bfloat16(v);
  }
}

// dpre[t, d] = dy * act'(pre) with pre recomputed; dw[d, j] += sum_t dpre * in_j   (atomic per block)
template <int TT>
__global__ void conv1d_bwd_pre_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ w,
                                      const bf16* __restrict__ init, const int* __restrict__ cu, int nseq,
                                      const bf16* __restrict__ dy, float* __restrict__ dpre, float* __restrict__ dw, int T,
                                      int D, int W, int act) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float wr[MAXW], gw[MAXW];
  for (int j = 0; j < W; ++j) { wr[j] = __bfloat162float(w[(long)d * W + j]); gw[j] = 0.f; }
  const int tb = blockIdx.y * TT;
  for (int t = tb; t < min(T, tb + TT); ++t) {
    const int s = seq_of(cu, nseq, t), a = cu[s], pos = t - a;
    float in[MAXW], acc = 0.f;
    for (int j = 0; j < W; ++j) { in[j] = conv_input(x, ldx, init, D, W, s, a, pos - (W - 1) + j, d); acc += wr[j] * in[j]; }
    float g = __bfloat162float(dy[(long)t * D + d]);
    if (act) {
      const float sg = sigmoidf(acc);
      g *= sg * (1.f + acc * (1.f - sg));
    }
    dpre[(long)t * D + d] = g;
    for (int j = 0; j < W; ++j) gw[j] += g * in[j];
  }
  if (dw != nullptr)
    for (int j = 0; j < W; ++j) atomicAdd(dw + (long)d * W + j, gw[j]);
}

// gradient of the virtual input at position pos: sum_j w[d,j] dpre[pos + (W-1) - j]  (+ dfin for the last W-1)
__device__ __forceinline__ float conv_dinput(const float* __restrict__ dpre, const float* wr, const bf16* __restrict__ dfin,
                                             int D, int W, int s, int a, int L, int pos, int d) {
  float acc = 0.f;
  for (int j = 0; j < W; ++j) {
    const int p = pos + (W - 1) - j;
    if (p >= 0 && p < L) acc += wr[j] * dpre[(long)(a + p) * D + d];
  }
  const int m = pos - (L - (W - 1));
  if (dfin != nullptr && m >= 0 && m < W - 1) acc += __bfloat162float(dfin[((long)s * D + d) * (W - 1) + m]);
  return acc;
}

template <int TT>
__global__ void conv1d_bwd_dx_kernel(const float* __restrict__ dpre, const bf16* __restrict__ w,
                                     const bf16* __restrict__ dfin, const int* __restrict__ cu, int nseq,
                                     bf16* __restrict__ dx, long lddx, int T, int D, int W) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float wr[MAXW];
  for (int j = 0; j < W; ++j) wr[j] = __bfloat162float(w[(long)d * W + j]);
  const int tb = blockIdx.y * TT;
  for (int t = tb; t < min(T, tb + TT); ++t) {
    const int s = seq_of(cu, nseq, t), a = cu[s], L = cu[s + 1] - a;
    dx[(long)t * lddx + d] = __float2bfloat16(conv_dinput(dpre, wr, dfin, D, W, s, a, L, t - a, d));
  }
}

__global__ void conv1d_bwd_dinit_kernel(const float* __restrict__ dpre, const bf16* __restrict__ w,
                                        const bf16* __restrict__ dfin, const int* __restrict__ cu, bf16* __restrict__ dinit,
                                        int D, int W) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (d >= D) return;
  float wr[MAXW];
  for (int j = 0; j < W; ++j) wr[j] = __bfloat162float(w[(long)d * W + j]);
  const int a = cu[s], L = cu[s + 1] - a;
  for (int m = 0; m < W - 1; ++m)
    dinit[((long)s * D + d) * (W - 1) + m] =
        __float2bfloat16(conv_dinput(dpre, wr, dfin, D, W, s, a, L, m - (W - 1), d));
}

// ---------------------------------------------------------------------------------------------- L2 norm
// rows = T * H; row (t, h) lives at base + t * ld + h * D.  y = x * rsqrt(sum x^2 + eps)
__global__ void l2norm_strided_fwd_kernel(const bf16* __restrict__ x, long ldx, bf16* __restrict__ y, long ldy,
                                          float* __restrict__ rnorm, long rows, int H, int D, float eps) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long t = row / H;
  const int h = (int)(row - t * H);
  const bf16* xp = x + t * ldx + (long)h * D;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) { const float v = __bfloat162float(xp[i]); ss += v * v; }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss + eps);
  if (lane == 0 && rnorm) rnorm[row] = r;
  bf16* yp = y + t * ldy + (long)h * D;
  for (int i = lane; i < D; i += 32) yp[i] = __float2bfloat16(__bfloat162float(xp[i]) * r);
}

// dx = r * (dy - y * (dy . y)),  y = x * r;  dy is fp32 (the recurrence's gradients), dx bf16 (strided)
__global__ void l2norm_strided_bwd_kernel(const float* __restrict__ dy, const bf16* __restrict__ x, long ldx,
                                          const float* __restrict__ rnorm, bf16* __restrict__ dx, long lddx, long rows,
                                          int H, int D) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long t = row / H;
  const int h = (int)(row - t * H);
  const bf16* xp = x + t * ldx + (long)h * D;
  const float* gp = dy + row * D;
  const float r = rnorm[row];
  float dot = 0.f;
  for (int i = lane; i < D; i += 32) dot += gp[i] * __bfloat162float(xp[i]) * r;
  dot = warp_sum(dot);
  bf16* dp = dx + t * lddx + (long)h * D;
  for (int i = lane; i < D; i += 32) {
    const float y = __bfloat162float(xp[i]) * r;
    dp[i] = __float2bfloat16(r * (gp[i] - y * dot));
  }
}

// ----------------------------------------------------------------------------------- gated RMSNorm backward
// y = silu(z) * n * w,  n = o * rstd,  rstd = rsqrt(mean(o^2) + eps) per row (token, head)
__global__ void gated_rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ o, const bf16* __restrict__ z,
                                         long ldz, int H, const float* __restrict__ w, bf16* __restrict__ d_o,
                                         bf16* __restrict__ dz, long lddz, float* __restrict__ dw, long rows, int D,
                                         float eps) {
  extern __shared__ float dw_s[];      // D floats per CTA
  for (int i = threadIdx.x; i < D; i += blockDim.x) dw_s[i] = 0.f;
  __syncthreads();
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row < rows) {
    const long t = row / H;
    const int h = (int)(row - t * H);
    const bf16* op = o + row * D;
    const bf16* gp = dy + row * D;
    const bf16* zp = z + t * ldz + (long)h * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) { const float v = __bfloat162float(op[i]); ss += v * v; }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)D + eps);
    float dot = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float zz = __bfloat162float(zp[i]), sg = sigmoidf(zz);
      const float n = __bfloat162float(op[i]) * r;
      dot += __bfloat162float(gp[i]) * zz * sg * w[i] * n;
    }
    dot = warp_sum(dot) / (float)D;
    bf16* dop = d_o + row * D;
    bf16* dzp = dz + t * lddz + (long)h * D;
    for (int i = lane; i < D; i += 32) {
      const float zz = __bfloat162float(zp[i]), sg = sigmoidf(zz), gz = zz * sg;
      const float n = __bfloat162float(op[i]) * r;
      const float g = __bfloat162float(gp[i]);
      const float dn = g * gz * w[i];
      dop[i] = __float2bfloat16(r * (dn - n * dot));
      dzp[i] = __float2bfloat16(g * n * w[i] * sg * (1.f + zz * (1.f - sg)));
      atomicAdd(&dw_s[i], g * gz * n);
    }
  }
  __syncthreads();
  if (dw != nullptr)
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(dw + i, dw_s[i]);
}

// ------------------------------------------------------------------------------------------ top-p sampler
// One CTA per row.  p = softmax(logits / temperature); find by bisection the largest threshold tau such that the mass
// of {p_i >= tau} is still >= top_p (the nucleus), then draw from the renormalised nucleus with the row's uniform u.
__global__ void top_p_kernel(const bf16* __restrict__ logits, const float* __restrict__ u, long* __restrict__ out, int V,
                             float top_p, float inv_temp) {
  extern __shared__ float sh[];        // blockDim.x floats
  const long row = blockIdx.x;
  const bf16* z = logits + row * V;
  const int tid = threadIdx.x, nt = blockDim.x;
  auto block_reduce = [&](float x, bool is_max) {
    sh[tid] = x;
    __syncthreads();
    for (int s = nt >> 1; s > 0; s >>= 1) {
      if (tid < s) sh[tid] = is_max ? fmaxf(sh[tid], sh[tid + s]) : sh[tid] + sh[tid + s];
      __syncthreads();
    }
    const float r = sh[0];
    __syncthreads();
    return r;
  };
  float mx = -INFINITY;
  for (int i = tid; i < V; i += nt) mx = fmaxf(mx, __bfloat162float(z[i]) * inv_temp);
  mx = block_reduce(mx, true);
  float sum = 0.f;
  for (int i = tid; i < V; i += nt) sum += __expf(__bfloat162float(z[i]) * inv_temp - mx);
  sum = block_reduce(sum, false);
  const float inv = 1.f / sum;
  float lo = 0.f, hi = 1.f;            // mass(p >= lo) >= top_p  >  mass(p >= hi) is kept as the invariant
  for (int it = 0; it < 24; ++it) {
    const float mid = 0.5f * (lo + hi);
    float m = 0.f;
    for (int i = tid; i < V; i += nt) {
      const float p = __expf(__bfloat162float(z[i]) * inv_temp - mx) * inv;
      if (p >= mid) m += p;
    }
    m = block_reduce(m, false);
    if (m >= top_p) lo = mid; else hi = mid;
  }
  float mass = 0.f;
  for (int i = tid; i < V; i += nt) {
    const float p = __expf(__bfloat162float(z[i]) * inv_temp - mx) * inv;
    if (p >= lo) mass += p;
  }
  mass = block_reduce(mass, false);
  // sequential scan by thread 0 over the nucleus in index order (generation-time utility; V reads from L2)
  if (tid == 0) {
    const float target = u[row] * mass;
    float c = 0.f;
    long pick = -1, last = 0;
    for (int i = 0; i < V; ++i) {
      const float p = __expf(__bfloat162float(z[i]) * inv_temp - mx) * inv;
      if (p >= lo) {
        c += p;
        last = i;
        if (c >= target) { pick = i; break; }
      }
    }
    out[row] = pick >= 0 ? pick : last;
  }
}

}  // namespace

#define CHECK_LAUNCH()                                 \
  do {                                                 \
    cudaError_t e_ = cudaGetLastError();               \
    return e_ == cudaSuccess ? 0 : -400 - (int)e_;     \
  } while (0)


// ----------------------------------------------------------------------------------------- gate preparation
// Gated DeltaNet gates from the fused [b | a] projection (flextrain/ops/_kernels/gate_prep.py:29-80):
//   beta = sigmoid(b),   g = -exp(A_log) * softplus(a + dt_bias)          (per token and value head)
// and their backward:  db = dbeta * beta (1 - beta),  da = dg * (-exp(A_log)) * sigmoid(a + dt_bias),
//   dA_log[h] += sum_t dg * g,   d_dt_bias[h] += sum_t da.
// ba is the bf16 GEMM output (T, 2*HV); beta / g are fp32 (T, HV); dba is bf16 (T, 2*HV).
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__global__ void gate_prep_fwd_kernel(const __nv_bfloat16* __restrict__ ba, const float* __restrict__ dt_bias,
                                     const float* __restrict__ a_log, float* __restrict__ beta, float* __restrict__ g,
                                     long T, int HV) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * HV) return;
  const long t = i / HV;
  const int h = (int)(i - t * HV);
  const float b = __bfloat162float(ba[t * 2 * HV + h]);
  const float a = __bfloat162float(ba[t * 2 * HV + HV + h]) + dt_bias[h];
  beta[i] = 1.f / (1.f + __expf(-b));
  g[i] = -__expf(a_log[h]) * softplus_f(a);
}

// grid: blocks of 256 threads over heads x token slabs; each block reduces its slab's column sums in shared memory
__global__ void gate_prep_bwd_kernel(const __nv_bfloat16* __restrict__ ba, const float* __restrict__ dt_bias,
                                     const float* __restrict__ a_log, const float* __restrict__ g,
                                     const float* __restrict__ dbeta, const float* __restrict__ dg,
                                     __nv_bfloat16* __restrict__ dba, float* __restrict__ d_a_log,
                                     float* __restrict__ d_dt_bias, long T, int HV, int rows_per_block) {
  extern __shared__ float sh[];            // [2 * HV] column sums of this block
  for (int j = threadIdx.x; j < 2 * HV; j += blockDim.x) sh[j] = 0.f;
  __syncthreads();
  const long t0 = (long)blockIdx.x * rows_per_block;
  const long t1 = min(T, t0 + rows_per_block);
  for (long i = t0 * HV + threadIdx.x; i < t1 * HV; i += blockDim.x) {
    const long t = i / HV;
    const int h = (int)(i - t * HV);
    const float b = __bfloat162float(ba[t * 2 * HV + h]);
    const float a = __bfloat162float(ba[t * 2 * HV + HV + h]) + dt_bias[h];
    const float be = 1.f / (1.f + __expf(-b));
    const float dgi = dg[i];
    const float da = dgi * (-__expf(a_log[h])) * (1.f / (1.f + __expf(-a)));
    dba[t * 2 * HV + h] = __float2bfloat16(dbeta[i] * be * (1.f - be));
    dba[t * 2 * HV + HV + h] = __float2bfloat16(da);
    atomicAdd(&sh[h], dgi * g[i]);
    atomicAdd(&sh[HV + h], da);
  }
  __syncthreads();
  for (int j = threadIdx.x; j < HV; j += blockDim.x) {
    if (d_a_log) atomicAdd(d_a_log + j, sh[j]);
    if (d_dt_bias) atomicAdd(d_dt_bias + j, sh[HV + j]);
  }
}

extern "C" {

int ftb_gate_prep_fwd(const void* ba, const float* dt_bias, const float* a_log, float* beta, float* g, long T, int HV,
                      cudaStream_t s) {
  if (T == 0) return 0;
  const long n = T * HV;
  gate_prep_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const __nv_bfloat16*)ba, dt_bias, a_log, beta, g, T, HV);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - (int)e;
}

// d_a_log / d_dt_bias (HV fp32) are ACCUMULATED into (pass zeroed buffers for plain sums); either may be NULL.
int ftb_gate_prep_bwd(const void* ba, const float* dt_bias, const float* a_log, const float* g, const float* dbeta,
                      const float* dg, void* dba, float* d_a_log, float* d_dt_bias, long T, int HV, cudaStream_t s) {
  if (T == 0) return 0;
  if (HV > 4096) return -2;
  const int rows = 128;
  gate_prep_bwd_kernel<<<(unsigned)((T + rows - 1) / rows), 256, 2 * HV * sizeof(float), s>>>(
      (const __nv_bfloat16*)ba, dt_bias, a_log, g, dbeta, dg, (__nv_bfloat16*)dba, d_a_log, d_dt_bias, T, HV, rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - (int)e;
}

int ftb_conv1d_fwd(const void* x, long ldx, const void* w, const void* init, const int* cu, int nseq, void* y, void* fin,
                   int T, int D, int W, int act, cudaStream_t s) {
  if (W > MAXW || W < 2) return -2;
  if (T > 0) {
    dim3 grid((D + 127) / 128, (T + 63) / 64);
    conv1d_fwd_kernel<64><<<grid, 128, 0, s>>>((const bf16*)x, ldx, (const bf16*)w, (const bf16*)init, cu, nseq,
                                               (bf16*)y, T, D, W, act);
  }
  if (fin != nullptr && nseq > 0) {
    dim3 grid((D + 127) / 128, nseq);
    conv1d_state_kernel<<<grid, 128, 0, s>>>((const bf16*)x, ldx, (const bf16*)init, cu, (bf16*)fin, D, W);
  }
  CHECK_LAUNCH();
}

// dpre: (T, D) fp32 scratch; dw: (D, W) fp32 accumulated; dfin / dinit: (nseq, D, W-1) bf16 or null
int ftb_conv1d_bwd(const void* x, long ldx, const void* w, const void* init, const int* cu, int nseq, const void* dy,
                   const void* dfin, float* dpre, void* dx, long lddx, float* dw, void* dinit, int T, int D, int W,
                   int act, cudaStream_t s) {
  if (W > MAXW || W < 2) return -2;
  if (T > 0) {
    dim3 grid((D + 127) / 128, (T + 127) / 128);
    conv1d_bwd_pre_kernel<128><<<grid, 128, 0, s>>>((const bf16*)x, ldx, (const bf16*)w, (const bf16*)init, cu, nseq,
                                                    (const bf16*)dy, dpre, dw, T, D, W, act);
    dim3 grid2((D + 127) / 128, (T + 63) / 64);
    conv1d_bwd_dx_kernel<64><<<grid2, 128, 0, s>>>(dpre, (const bf16*)w, (const bf16*)dfin, cu, nseq, (bf16*)dx, lddx,
                                                   T, D, W);
  }
  if (dinit != nullptr && nseq > 0) {
    dim3 grid((D + 127) / 128, nseq);
    conv1d_bwd_dinit_kernel<<<grid, 128, 0, s>>>(dpre, (const bf16*)w, (const bf16*)dfin, cu, (bf16*)dinit, D, W);
  }
  CHECK_LAUNCH();
}

int ftb_l2norm_strided_fwd(const void* x, long ldx, void* y, long ldy, float* rnorm, long T, int H, int D, float eps,
                           cudaStream_t s) {
  const long rows = T * H;
  if (rows == 0) return 0;
  l2norm_strided_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const bf16*)x, ldx, (bf16*)y, ldy, rnorm, rows,
                                                                       H, D, eps);
  CHECK_LAUNCH();
}

int ftb_l2norm_strided_bwd(const float* dy, const void* x, long ldx, const float* rnorm, void* dx, long lddx, long T,
                           int H, int D, cudaStream_t s) {
  const long rows = T * H;
  if (rows == 0) return 0;
  l2norm_strided_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(dy, (const bf16*)x, ldx, rnorm, (bf16*)dx, lddx,
                                                                       rows, H, D);
  CHECK_LAUNCH();
}

int ftb_gated_rmsnorm_bwd(const void* dy, const void* o, const void* z, long ldz, int H, const float* w, void* d_o,
                          void* dz, long lddz, float* dw, long T, int D, float eps, cudaStream_t s) {
  const long rows = T * H;
  if (rows == 0) return 0;
  gated_rmsnorm_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, D * sizeof(float), s>>>(
      (const bf16*)dy, (const bf16*)o, (const bf16*)z, ldz, H, w, (bf16*)d_o, (bf16*)dz, lddz, dw, rows, D, eps);
  CHECK_LAUNCH();
}

int ftb_top_p(const void* logits, const float* u, long* out, int rows, int V, float top_p, float temperature,
              cudaStream_t s) {
  if (rows == 0) return 0;
  top_p_kernel<<<rows, 256, 256 * sizeof(float), s>>>((const bf16*)logits, u, out, V, top_p,
                                                      1.f / fmaxf(temperature, 1e-6f));
  CHECK_LAUNCH();
}

}  // extern "C"
