// Bandwidth-bound kernels for sm_100a: RMSNorm fwd/bwd (+residual-grad add, +re-emit), RoPE
// (rotate-half, partial, MRoPE), SwiGLU / GeGLU fwd/bwd, fused softmax cross-entropy, embedding
// gather / sorted scatter-add, multi-tensor AdamW, gated RMSNorm, L2 norm, top-k router.
// They replace the reference project's Triton kernels (flextrain/ops/_kernels/*.py). All use
// 16-byte vector accesses and keep a row in registers between the reduction and the write.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int NW>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < NW) ? sh[l] : 0.f;
  return warp_sum(t);
}
template <int NW>
__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < NW) ? sh[l] : -INFINITY;
  return warp_max(t);
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

// ----------------------------------------------------------------------------- RMSNorm
// One CTA (256 threads) walks rows; a row of up to 8*256*MAXV elements lives in registers.
constexpr int RN_THREADS = 256;
constexpr int RN_MAXV = 8;  // D <= 16384

template <int MAXV>
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_fwd_kernel(const bf16* __restrict__ x,
                                                                  const float* __restrict__ w, bf16* __restrict__ y,
                                                                  float* __restrict__ rstd_out, int T, int D,
                                                                  float eps) {
  __shared__ float sh[32];
  const int nv = D >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    uint4 v[MAXV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * RN_THREADS;
      if (i < nv) {
        v[j] = xr[i];
        float f[8];
        unpack8(v[j], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
      }
    }
    ss = block_sum<RN_THREADS / 32>(ss, sh);
    const float r = rsqrtf(ss / (float)D + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = r;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * D);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * RN_THREADS;
      if (i < nv) {
        float f[8];
        unpack8(v[j], f);
        if (w) {
          const float4 w0 = reinterpret_cast<const float4*>(w)[2 * i];
          const float4 w1 = reinterpret_cast<const float4*>(w)[2 * i + 1];
          f[0] *= r * w0.x; f[1] *= r * w0.y; f[2] *= r * w0.z; f[3] *= r * w0.w;
          f[4] *= r * w1.x; f[5] *= r * w1.y; f[6] *= r * w1.z; f[7] *= r * w1.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] *= r;
        }
        yr[i] = pack8(f);
      }
    }
  }
}

// dx = (g - xhat * mean(g . xhat)) * rstd, g = dy * w; optional dx += dx_add (residual gradient),
// optional y_out = xhat * w (forward output re-emitted for the deferred weight-gradient GEMMs);
// partial dw[blockIdx.x, :] = sum over this CTA's rows of dy * xhat (fp32), reduced by a second kernel.
template <int MAXV>
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_bwd_kernel(const bf16* __restrict__ dy,
                                                                  const bf16* __restrict__ x,
                                                                  const float* __restrict__ w,
                                                                  const float* __restrict__ rstd,
                                                                  const bf16* __restrict__ dx_add,
                                                                  bf16* __restrict__ dx, bf16* __restrict__ y_out,
                                                                  float* __restrict__ dw_partial, int T, int D) {
  __shared__ float sh[32];
  const int nv = D >> 3;
  float dwacc[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[j][e] = 0.f;

  // The next row's operands are requested before the current row's block-wide reduction, so its DRAM latency hides
  // behind the two barriers and the arithmetic of this row (the kernel is latency-bound otherwise: one row in flight
  // per CTA).
  uint4 nx[MAXV], ng[MAXV], na[MAXV];
  float nr = 0.f;
  auto prefetch = [&](int rw) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)rw * D);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)rw * D);
    nr = rstd[rw];
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * RN_THREADS;
      if (i < nv) {
        nx[j] = xr[i];
        ng[j] = dyr[i];
        if (dx_add) na[j] = reinterpret_cast<const uint4*>(dx_add + (size_t)rw * D)[i];
      }
    }
  };
  constexpr bool AHEAD = MAXV <= 2;          // wider rows would halve the CTAs per SM with two rows in registers
  if (AHEAD && blockIdx.x < T) prefetch(blockIdx.x);
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    if (!AHEAD) prefetch(row);
    const float r = nr;
    uint4 xv[MAXV], gv[MAXV], av[MAXV];
#pragma unroll
    for (int j = 0; j < MAXV; ++j) { xv[j] = nx[j]; gv[j] = ng[j]; av[j] = na[j]; }
    if (AHEAD && row + (int)gridDim.x < T) prefetch(row + gridDim.x);
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * RN_THREADS;
      if (i < nv) {
        float xf[8], gf[8], wf[8];
        unpack8(xv[j], xf);
        unpack8(gv[j], gf);
        if (w) {
          const float4 w0 = reinterpret_cast<const float4*>(w)[2 * i];
          const float4 w1 = reinterpret_cast<const float4*>(w)[2 * i + 1];
          wf[0] = w0.x; wf[1] = w0.y; wf[2] = w0.z; wf[3] = w0.w; wf[4] = w1.x; wf[5] = w1.y; wf[6] = w1.z; wf[7] = w1.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) wf[e] = 1.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = xf[e] * r;
          dwacc[j][e] += gf[e] * xh;
          dot += gf[e] * wf[e] * xh;
        }
      }
    }
    dot = block_sum<RN_THREADS / 32>(dot, sh) / (float)D;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * D);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * RN_THREADS;
      if (i < nv) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xv[j], xf);
        unpack8(gv[j], gf);
        if (w) {
          const float4 w0 = reinterpret_cast<const float4*>(w)[2 * i];
          const float4 w1 = reinterpret_cast<const float4*>(w)[2 * i + 1];
          wf[0] = w0.x; wf[1] = w0.y; wf[2] = w0.z; wf[3] = w0.w; wf[4] = w1.x; wf[5] = w1.y; wf[6] = w1.z; wf[7] = w1.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) wf[e] = 1.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (gf[e] * wf[e] - xf[e] * r * dot) * r;
        if (dx_add) {
          float a[8];
          unpack8(av[j], a);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += a[e];
        }
        dxr[i] = pack8(o);
        if (y_out) {
          float yv[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) yv[e] = xf[e] * r * wf[e];
          reinterpret_cast<uint4*>(y_out + (size_t)row * D)[i] = pack8(yv);
        }
      }
    }
  }
  if (dw_partial) {
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int i = threadIdx.x + j * RN_THREADS;
      if (i < nv) {
        float* o = dw_partial + (size_t)blockIdx.x * D + i * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = dwacc[j][e];
      }
    }
  }
}

__global__ void colsum_accum_kernel(const float* __restrict__ partial, float* __restrict__ out, int P, int D,
                                    int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[(size_t)p * D + c];
  out[c] = accumulate ? out[c] + s : s;
}

// Small-D (per-head) RMSNorm: one warp per row of D <= 512 elements (QK-norm, D = head_dim).
__global__ void rmsnorm_small_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ w, bf16* __restrict__ y,
                                         float* __restrict__ rstd_out, long rows, int D, int heads_w, float eps) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const bf16* xr = x + row * D;
  float ss = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 t = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
    ss += t.x * t.x + t.y * t.y;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)D + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = r;
  // heads_w > 1: weight has one row per head (full-row QK-norm over H*hd is handled by the big kernel).
  const float* wr = w ? w + (heads_w > 1 ? (row % heads_w) * D : 0) : nullptr;
  bf16* yr = y + row * D;
  for (int i = lane * 2; i < D; i += 64) {
    float2 t = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
    t.x *= r * (wr ? wr[i] : 1.f);
    t.y *= r * (wr ? wr[i + 1] : 1.f);
    *reinterpret_cast<bf162*>(yr + i) = __floats2bfloat162_rn(t.x, t.y);
  }
}

__global__ void rmsnorm_small_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                         const float* __restrict__ w, const float* __restrict__ rstd,
                                         bf16* __restrict__ dx, float* __restrict__ dw, long rows, int D) {
  // One warp per row, grid-stride over rows.  dw (D,) partial sums stay in registers while a warp walks its rows
  // (D <= 512: 8 pairs per lane), are combined across the CTA's warps in shared memory and leave with ONE atomic per
  // element per CTA; a per-row atomic on D hot addresses serialises the whole grid.
  constexpr int MAXP = 8;
  extern __shared__ float dw_sh[];                 // D floats
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  float2 acc[MAXP];
#pragma unroll
  for (int p = 0; p < MAXP; ++p) acc[p] = make_float2(0.f, 0.f);
  for (int i = threadIdx.x; i < D; i += blockDim.x) dw_sh[i] = 0.f;
  __syncthreads();
  for (long row = (long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += (long)gridDim.x * wpb) {
    const bf16* xr = x + row * D;
    const bf16* gr = dy + row * D;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane * 2; i < D; i += 64) {
      const float2 xv = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
      const float2 gv = __bfloat1622float2(*reinterpret_cast<const bf162*>(gr + i));
      const float w0 = w ? w[i] : 1.f, w1 = w ? w[i + 1] : 1.f;
      dot += gv.x * w0 * xv.x * r + gv.y * w1 * xv.y * r;
    }
    dot = warp_sum(dot) / (float)D;
    bf16* dxr = dx + row * D;
#pragma unroll
    for (int p = 0; p < MAXP; ++p) {
      const int i = lane * 2 + p * 64;
      if (i < D) {
        const float2 xv = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
        const float2 gv = __bfloat1622float2(*reinterpret_cast<const bf162*>(gr + i));
        const float w0 = w ? w[i] : 1.f, w1 = w ? w[i + 1] : 1.f;
        const float o0 = (gv.x * w0 - xv.x * r * dot) * r;
        const float o1 = (gv.y * w1 - xv.y * r * dot) * r;
        *reinterpret_cast<bf162*>(dxr + i) = __floats2bfloat162_rn(o0, o1);
        acc[p].x += gv.x * xv.x * r;
        acc[p].y += gv.y * xv.y * r;
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int p = 0; p < MAXP; ++p) {
      const int i = lane * 2 + p * 64;
      if (i < D) {
        atomicAdd(&dw_sh[i], acc[p].x);
        atomicAdd(&dw_sh[i + 1], acc[p].y);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(dw + i, dw_sh[i]);
  }
}

// -------------------------------------------------------------------------------- RoPE
// out[t,h,:] = R(pos_t) x[t,h,:] over rotate-half pairs (i, i + rot/2), i < rot/2; channels past
// 2*half_rot are copied. x / out are (T, H, hd) with independent token strides (in place when equal),
// so Q and K can be rotated straight out of a fused QKV projection buffer. positions: (T) or (T,3).
__global__ void rope_kernel(const bf16* __restrict__ x, long in_stride, bf16* __restrict__ out, long out_stride,
                            const int* __restrict__ pos, const float* __restrict__ inv_freq, int T, int H, int hd,
                            int half_rot, int inverse, int pos_stride, int sec_h, int sec_w) {
  const int t = blockIdx.x;
  const int* pr = pos + (size_t)t * pos_stride;
  const int half_hd = hd >> 1;
  for (int idx = threadIdx.x; idx < H * half_hd; idx += blockDim.x) {
    const int h = idx / half_hd, i = idx - h * half_hd;
    const bf16* p = x + (size_t)t * in_stride + (size_t)h * hd;
    bf16* o = out + (size_t)t * out_stride + (size_t)h * hd;
    if (i < half_rot) {
      int axis = 0;
      if (pos_stride == 3) {
        // interleaved MRoPE: slot i takes axis (i % 3) while it lies inside that axis' section span
        const int a = i % 3;
        if (a == 1 && i < 3 * sec_h) axis = 1;
        if (a == 2 && i < 3 * sec_w) axis = 2;
      }
      const float ang = (float)pr[axis] * inv_freq[i];
      float s, c;
      sincosf(ang, &s, &c);
      if (inverse) s = -s;
      const float a = __bfloat162float(p[i]), b = __bfloat162float(p[i + half_rot]);
      o[i] = __float2bfloat16(a * c - b * s);
      o[i + half_rot] = __float2bfloat16(b * c + a * s);
    } else if (o != p) {
      // pass-through tail (partial rotary): channels [2*half_rot, hd)
      const int c0 = 2 * half_rot + 2 * (i - half_rot);
      o[c0] = p[c0];
      o[c0 + 1] = p[c0 + 1];
    }
  }
}

// Full-rotary fast path (one position axis, rot == hd, hd % 16 == 0, 16-byte aligned rows): one block per token.
// The hd/2 (sin, cos) pairs of the token are computed once into shared memory and reused by every head; each thread
// then rotates 8 pairs of one head with two 16-byte loads and two 16-byte stores.
__global__ void rope_full_vec_kernel(const bf16* __restrict__ x, long in_stride, bf16* __restrict__ out, long out_stride,
                                     const int* __restrict__ pos, const float* __restrict__ inv_freq, int T, int H,
                                     int hd, int inverse) {
  extern __shared__ float sc[];              // [half] sin, [half] cos
  const int t = blockIdx.x;
  const int half = hd >> 1;
  const float pf = (float)pos[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf(pf * inv_freq[i], &sn, &cs);
    sc[i] = inverse ? -sn : sn;
    sc[half + i] = cs;
  }
  __syncthreads();
  const int per_head = half >> 3;            // 8-pair chunks per head
  const bf16* xr = x + (size_t)t * in_stride;
  bf16* orow = out + (size_t)t * out_stride;
  for (int idx = threadIdx.x; idx < H * per_head; idx += blockDim.x) {
    const int h = idx / per_head, c = (idx - h * per_head) << 3;
    const uint4 ua = *reinterpret_cast<const uint4*>(xr + (size_t)h * hd + c);
    const uint4 ub = *reinterpret_cast<const uint4*>(xr + (size_t)h * hd + half + c);
    float a[8], b[8], ra[8], rb[8];
    unpack8(ua, a);
    unpack8(ub, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sn = sc[c + e], cs = sc[half + c + e];
      ra[e] = a[e] * cs - b[e] * sn;
      rb[e] = b[e] * cs + a[e] * sn;
    }
    *reinterpret_cast<uint4*>(orow + (size_t)h * hd + c) = pack8(ra);
    *reinterpret_cast<uint4*>(orow + (size_t)h * hd + half + c) = pack8(rb);
  }
}

// ------------------------------------------------------------------------ SwiGLU / GeGLU
__device__ __forceinline__ void act_and_grad(float g, int kind, float& a, float& da) {
  if (kind == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    a = g * s;
    da = s * (1.f + g * (1.f - s));
  } else {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float t = tanhf(k0 * (g + k1 * g * g * g));
    a = 0.5f * g * (1.f + t);
    da = 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
  }
}

// gate / up may be column slices of one (T, ld) buffer (a fused [gate | up] projection output).
__global__ void glu_fwd_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up, bf16* __restrict__ out,
                               long T, int F, int ld_in, int ld_out, int kind) {
  const long nvec = T * (F >> 3);
  for (long v = (long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long)gridDim.x * blockDim.x) {
    const long t = v / (F >> 3);
    const int c = (int)(v - t * (F >> 3)) << 3;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gate + t * ld_in + c), g);
    unpack8(*reinterpret_cast<const uint4*>(up + t * ld_in + c), u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float a, da;
      act_and_grad(g[e], kind, a, da);
      o[e] = a * u[e];
    }
    *reinterpret_cast<uint4*>(out + t * ld_out + c) = pack8(o);
  }
}

__global__ void glu_bwd_kernel(const bf16* __restrict__ dact, const bf16* __restrict__ gate,
                               const bf16* __restrict__ up, bf16* __restrict__ dgate, bf16* __restrict__ dup,
                               bf16* __restrict__ act_out, long T, int F, int ld_in, int ld_d, int ld_act, int kind) {
  const long nvec = T * (F >> 3);
  for (long v = (long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long)gridDim.x * blockDim.x) {
    const long t = v / (F >> 3);
    const int c = (int)(v - t * (F >> 3)) << 3;
    float g[8], u[8], d[8], og[8], ou[8], oa[8];
    unpack8(*reinterpret_cast<const uint4*>(gate + t * ld_in + c), g);
    unpack8(*reinterpret_cast<const uint4*>(up + t * ld_in + c), u);
    unpack8(*reinterpret_cast<const uint4*>(dact + t * ld_act + c), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float a, da;
      act_and_grad(g[e], kind, a, da);
      og[e] = d[e] * u[e] * da;
      ou[e] = d[e] * a;
      oa[e] = a * u[e];
    }
    *reinterpret_cast<uint4*>(dgate + t * ld_d + c) = pack8(og);
    *reinterpret_cast<uint4*>(dup + t * ld_d + c) = pack8(ou);
    if (act_out) *reinterpret_cast<uint4*>(act_out + t * ld_act + c) = pack8(oa);
  }
}

// MoE expert backward through the gated activation with the router weight folded in, one CTA per expert-major row
// (the reference's swiglu_bwd_weighted kernel, flextrain/ops/_kernels/moe.py:77-145):
//   act = glu(gate, up);  d = w_row * dact_u;  dgate, dup from d;  act_w = w_row * act (left operand of the down-proj
//   weight gradient, so dy needs no separate scaling pass);  dw_row = sum_c dact_u * act (router-weight gradient).
__global__ void glu_bwd_weighted_kernel(const bf16* __restrict__ dact, const bf16* __restrict__ gate,
                                        const bf16* __restrict__ up, const float* __restrict__ w_row,
                                        bf16* __restrict__ dgate, bf16* __restrict__ dup, bf16* __restrict__ act_w,
                                        float* __restrict__ dw_row, int F, int ld_in, int ld_d, int kind) {
  __shared__ float red[32];
  const long t = blockIdx.x;
  const float wr = w_row[t];
  float dot = 0.f;
  for (int c = threadIdx.x << 3; c < F; c += blockDim.x << 3) {
    float g[8], u[8], d[8], og[8], ou[8], oa[8];
    unpack8(*reinterpret_cast<const uint4*>(gate + t * ld_in + c), g);
    unpack8(*reinterpret_cast<const uint4*>(up + t * ld_in + c), u);
    unpack8(*reinterpret_cast<const uint4*>(dact + t * (long)F + c), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float a, da;
      act_and_grad(g[e], kind, a, da);
      const float act = a * u[e];
      dot += d[e] * act;
      const float dd = d[e] * wr;
      og[e] = dd * u[e] * da;
      ou[e] = dd * a;
      oa[e] = act * wr;
    }
    *reinterpret_cast<uint4*>(dgate + t * ld_d + c) = pack8(og);
    *reinterpret_cast<uint4*>(dup + t * ld_d + c) = pack8(ou);
    *reinterpret_cast<uint4*>(act_w + t * (long)F + c) = pack8(oa);
  }
  dot = warp_sum(dot);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) dw_row[t] = v;
  }
}

// ----------------------------------------------------------------- softmax cross-entropy
// One CTA per row. Pass 1: online max / sum over V (bf16 logits). Pass 2: logits <- grad_scale *
// (softmax - onehot) in place (the second read hits L2). Optional tanh soft-cap chained through.
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS) softmax_ce_kernel(bf16* __restrict__ logits,
                                                                 const long* __restrict__ targets,
                                                                 const float* __restrict__ loss_mask,
                                                                 float* __restrict__ loss, int T, int V, long ld,
                                                                 float grad_scale, float softcap, long ignore_index) {
  __shared__ float sh[32];
  const int row = blockIdx.x;
  bf16* z = logits + (size_t)row * ld;
  const long tgt = targets[row];
  bool valid = tgt != ignore_index && tgt >= 0 && tgt < V;
  if (loss_mask && loss_mask[row] <= 0.f) valid = false;
  const int nv = V >> 3;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  if (!valid) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < nv; i += CE_THREADS) reinterpret_cast<uint4*>(z)[i] = zero;
    for (int i = (nv << 3) + threadIdx.x; i < V; i += CE_THREADS) z[i] = __float2bfloat16(0.f);
    if (threadIdx.x == 0) loss[row] = 0.f;
    return;
  }
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(z)[i], f);
    float lm = -INFINITY;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (softcap > 0.f) f[e] = softcap * tanhf(f[e] * inv_cap);
      lm = fmaxf(lm, f[e]);
    }
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += __expf(f[e] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = (nv << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    float f = __bfloat162float(z[i]);
    if (softcap > 0.f) f = softcap * tanhf(f * inv_cap);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  const float gm = block_max<CE_THREADS / 32>(m, sh);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum<CE_THREADS / 32>(s, sh);
  const float lse = gm + logf(gs);
  if (threadIdx.x == 0) {
    float zt = __bfloat162float(z[tgt]);
    if (softcap > 0.f) zt = softcap * tanhf(zt * inv_cap);
    loss[row] = lse - zt;
  }
  __syncthreads();  // the target logit is read before anyone overwrites it
  const int tv = (int)(tgt >> 3), te = (int)(tgt & 7);
  for (int i = threadIdx.x; i < nv; i += CE_THREADS) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(z)[i], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float zc = f[e], dcap = 1.f;
      if (softcap > 0.f) {
        const float t = tanhf(f[e] * inv_cap);
        zc = softcap * t;
        dcap = 1.f - t * t;
      }
      float p = __expf(zc - lse);
      if (i == tv && e == te) p -= 1.f;
      f[e] = p * grad_scale * dcap;
    }
    reinterpret_cast<uint4*>(z)[i] = pack8(f);
  }
  for (int i = (nv << 3) + threadIdx.x; i < V; i += CE_THREADS) {
    float f = __bfloat162float(z[i]), dcap = 1.f;
    if (softcap > 0.f) {
      const float t = tanhf(f * inv_cap);
      f = softcap * t;
      dcap = 1.f - t * t;
    }
    float p = __expf(f - lse);
    if (i == tgt) p -= 1.f;
    z[i] = __float2bfloat16(p * grad_scale * dcap);
  }
}

// ----------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const long* __restrict__ tokens, const bf16* __restrict__ table,
                                     bf16* __restrict__ out, int T, int D, float scale) {
  const int t = blockIdx.x;
  const long tok = tokens[t];
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)tok * D);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * D);
  for (int i = threadIdx.x; i < (D >> 3); i += blockDim.x) {
    uint4 v = src[i];
    if (scale != 1.f) {
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= scale;
      v = pack8(f);
    }
    dst[i] = v;
  }
}

// Sorted scatter-add: sorted_tok ascending, order[i] = original row of sorted position i.
// The CTA at the head of each run sums the run in fp32 and adds it to the gradient row once.
__global__ void embedding_bwd_kernel(const long* __restrict__ sorted_tok, const long* __restrict__ order,
                                     const bf16* __restrict__ dy, void* __restrict__ grad, int T, int D, float scale,
                                     int grad_fp32) {
  const int i0 = blockIdx.x;
  const long tok = sorted_tok[i0];
  if (i0 > 0 && sorted_tok[i0 - 1] == tok) return;
  int i1 = i0 + 1;
  while (i1 < T && sorted_tok[i1] == tok) ++i1;
  for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = i0; i < i1; ++i) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(dy + (size_t)order[i] * D)[c], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    if (grad_fp32) {
      float* g = reinterpret_cast<float*>(grad) + (size_t)tok * D + c * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] += acc[e] * scale;
    } else {
      uint4* g = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(grad) + (size_t)tok * D) + c;
      float f[8];
      unpack8(*g, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] += acc[e] * scale;
      *g = pack8(f);
    }
  }
}

// --------------------------------------------------------------------------- AdamW
// Multi-tensor: one launch updates up to ADAM_MAX tensors (a whole layer). dtype codes: 0 bf16, 1 fp32.
constexpr int ADAM_MAX = 24;
struct AdamTensor {
  void* p; const void* g; void* m; void* v;
  long n;
  long block_start;  // first block of this tensor in the flattened grid
  float lr, wd;
  int p_dt, g_dt, s_dt, pad;
};
struct AdamArgs {
  AdamTensor t[ADAM_MAX];
  int count;
  float beta1, beta2, eps, bc1, bc2, grad_scale;
};
constexpr int ADAM_THREADS = 256;
constexpr int ADAM_PER_BLOCK = ADAM_THREADS * 8;

__device__ __forceinline__ float ld_any(const void* p, long i, int dt) {
  return dt ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void st_any(void* p, long i, int dt, float v) {
  if (dt) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<bf16*>(p)[i] = __float2bfloat16(v);
}

__global__ void __launch_bounds__(ADAM_THREADS) adamw_kernel(const __grid_constant__ AdamArgs a) {
  int ti = 0;
#pragma unroll 1
  for (int i = 1; i < a.count; ++i)
    if ((long)blockIdx.x >= a.t[i].block_start) ti = i;
  const AdamTensor& t = a.t[ti];
  const long base = ((long)blockIdx.x - t.block_start) * ADAM_PER_BLOCK;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const long i = base + threadIdx.x + (long)j * ADAM_THREADS;
    if (i < t.n) {
      float p = ld_any(t.p, i, t.p_dt);
      const float g = ld_any(t.g, i, t.g_dt) * a.grad_scale;
      float m = ld_any(t.m, i, t.s_dt), v = ld_any(t.v, i, t.s_dt);
      p -= t.lr * t.wd * p;
      m = a.beta1 * m + (1.f - a.beta1) * g;
      v = a.beta2 * v + (1.f - a.beta2) * g * g;
      p -= t.lr * (m / a.bc1) / (sqrtf(v / a.bc2) + a.eps);
      st_any(t.p, i, t.p_dt, p);
      st_any(t.m, i, t.s_dt, m);
      st_any(t.v, i, t.s_dt, v);
    }
  }
}

// ------------------------------------------------------------------- gated RMSNorm / L2
__global__ void gated_rmsnorm_fwd_kernel(const bf16* __restrict__ o, const bf16* __restrict__ z,
                                         const float* __restrict__ w, bf16* __restrict__ y, long rows, int D,
                                         float eps) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float v = __bfloat162float(o[row * D + i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)D + eps);
  for (int i = lane; i < D; i += 32) {
    const float v = __bfloat162float(o[row * D + i]) * r * w[i];
    const float g = __bfloat162float(z[row * D + i]);
    y[row * D + i] = __float2bfloat16(v * g / (1.f + __expf(-g)));
  }
}

__global__ void l2norm_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, float* __restrict__ rnorm,
                                  long rows, int D, float eps) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float v = __bfloat162float(x[row * D + i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss + eps);
  if (lane == 0 && rnorm) rnorm[row] = r;
  for (int i = lane; i < D; i += 32) y[row * D + i] = __float2bfloat16(__bfloat162float(x[row * D + i]) * r);
}

// ------------------------------------------------------------------------- MoE routing
// Top-k by iterative arg-max (lowest index wins ties), softmax over the k picks (mode 0) or
// full softmax then top-k (mode 1). One warp per token; E <= 256.
__global__ void topk_route_kernel(const bf16* __restrict__ logits, float* __restrict__ weights,
                                  int* __restrict__ experts, int T, int E, int K, int mode) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  float v[8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + j * 32;
    v[j] = e < E ? __bfloat162float(logits[(size_t)t * E + e]) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  if (mode == 1) {
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = (lane + j * 32 < E) ? __expf(v[j] - mx) : -INFINITY;
      if (lane + j * 32 < E) s += v[j];
    }
    s = warp_sum(s);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (lane + j * 32 < E) v[j] /= s;
  }
  float pick_v[16];
  float top = 0.f;
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY;
    int bi = 1 << 30;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + j * 32;
      if (v[j] > bv) { bv = v[j]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (k == 0) top = bv;
    pick_v[k] = bv;
    if ((bi & 31) == lane) v[bi >> 5] = -INFINITY;
    if (lane == 0) experts[(size_t)t * K + k] = bi;
  }
  if (lane == 0) {
    if (mode == 0) {
      float s = 0.f;
      for (int k = 0; k < K; ++k) { pick_v[k] = __expf(pick_v[k] - top); s += pick_v[k]; }
      for (int k = 0; k < K; ++k) weights[(size_t)t * K + k] = pick_v[k] / s;
    } else {
      for (int k = 0; k < K; ++k) weights[(size_t)t * K + k] = pick_v[k];
    }
  }
}

// Row gather/scatter for MoE dispatch: out[i, :] = in[idx[i], :] * (w ? w[i] : 1).
__global__ void gather_rows_kernel(const bf16* __restrict__ in, const int* __restrict__ idx,
                                   const float* __restrict__ w, bf16* __restrict__ out, long rows, int D, int idx_div) {
  const long r = blockIdx.x;
  if (r >= rows) return;
  const int raw = idx[r];
  if (raw < 0) {  // padding row of an expert-major layout
    for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x)
      reinterpret_cast<uint4*>(out + r * D)[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const long src = raw / idx_div;
  const float s = w ? w[r] : 1.f;
  for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) {
    uint4 v = reinterpret_cast<const uint4*>(in + src * D)[c];
    if (w) {
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= s;
      v = pack8(f);
    }
    reinterpret_cast<uint4*>(out + r * D)[c] = v;
  }
}

// Combine: out[t, :] = resid[t, :] + sum_k w[t,k] * y[inv[t*K+k], :]  (fp32 accumulation).
__global__ void moe_combine_kernel(const bf16* __restrict__ y, const int* __restrict__ inv,
                                   const float* __restrict__ w, const bf16* __restrict__ resid,
                                   bf16* __restrict__ out, int T, int K, int D) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (resid) unpack8(reinterpret_cast<const uint4*>(resid + (size_t)t * D)[c], acc);
    for (int k = 0; k < K; ++k) {
      const long src = inv[(size_t)t * K + k];
      const float wk = w ? w[(size_t)t * K + k] : 1.f;
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(y + src * D)[c], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += wk * f[e];
    }
    reinterpret_cast<uint4*>(out + (size_t)t * D)[c] = pack8(acc);
  }
}

}  // namespace

#define CHECK_LAUNCH()                                   \
  do {                                                   \
    cudaError_t e_ = cudaGetLastError();                 \
    return e_ == cudaSuccess ? 0 : -400 - (int)e_;       \
  } while (0)

static int grid_rows(long rows, int cap) { return (int)(rows < cap ? rows : cap); }

extern "C" {

int ftb_rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd, int T, int D, float eps,
                    cudaStream_t s) {
  if (T == 0) return 0;
  if (D % 8 || D > 8 * RN_THREADS * RN_MAXV) return -2;
  const int nv = D / 8;
  if (nv <= 2 * RN_THREADS)
    rmsnorm_fwd_kernel<2><<<grid_rows(T, 148 * 8), RN_THREADS, 0, s>>>((const bf16*)x, w, (bf16*)y, rstd, T, D, eps);
  else if (nv <= 4 * RN_THREADS)
    rmsnorm_fwd_kernel<4><<<grid_rows(T, 148 * 8), RN_THREADS, 0, s>>>((const bf16*)x, w, (bf16*)y, rstd, T, D, eps);
  else
    rmsnorm_fwd_kernel<8><<<grid_rows(T, 148 * 8), RN_THREADS, 0, s>>>((const bf16*)x, w, (bf16*)y, rstd, T, D, eps);
  CHECK_LAUNCH();
}

// dw_partial: fp32 workspace of (ftb_rmsnorm_bwd_blocks(T) * D); dw (fp32, D) accumulated if dw != null.
int ftb_rmsnorm_bwd_blocks(int T) { return grid_rows(T, 148 * 4); }
int ftb_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, const void* dx_add, void* dx,
                    void* y_out, float* dw_partial, float* dw, int dw_accumulate, int T, int D, cudaStream_t s) {
  if (T == 0) return 0;
  if (D % 8 || D > 8 * RN_THREADS * RN_MAXV) return -2;
  const int blocks = ftb_rmsnorm_bwd_blocks(T);
  const int nv = D / 8;
#define FTB_RN_BWD(MV)                                                                                              \
  rmsnorm_bwd_kernel<MV><<<blocks, RN_THREADS, 0, s>>>((const bf16*)dy, (const bf16*)x, w, rstd, (const bf16*)dx_add, \
                                                       (bf16*)dx, (bf16*)y_out, dw ? dw_partial : nullptr, T, D)
  if (nv <= 2 * RN_THREADS) FTB_RN_BWD(2);
  else if (nv <= 4 * RN_THREADS) FTB_RN_BWD(4);
  else FTB_RN_BWD(8);
#undef FTB_RN_BWD
  if (dw) colsum_accum_kernel<<<(D + 255) / 256, 256, 0, s>>>(dw_partial, dw, blocks, D, dw_accumulate);
  CHECK_LAUNCH();
}

int ftb_rmsnorm_small_fwd(const void* x, const float* w, void* y, float* rstd, long rows, int D, int heads_w,
                          float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  if (D % 2) return -2;
  rmsnorm_small_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const bf16*)x, w, (bf16*)y, rstd, rows, D,
                                                                       heads_w, eps);
  CHECK_LAUNCH();
}
int ftb_rmsnorm_small_bwd(const void* dy, const void* x, const float* w, const float* rstd, void* dx, float* dw,
                          long rows, int D, cudaStream_t s) {
  if (rows == 0) return 0;
  if (D % 2 || D > 512) return -2;
  long blocks = (rows + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  rmsnorm_small_bwd_kernel<<<(unsigned)blocks, 256, D * sizeof(float), s>>>((const bf16*)dy, (const bf16*)x, w, rstd,
                                                                            (bf16*)dx, dw, rows, D);
  CHECK_LAUNCH();
}

int ftb_rope(const void* x, long in_stride, void* out, long out_stride, const int* pos, const float* inv_freq,
             int T, int H, int hd, int half_rot, int inverse, int pos_stride, int sec_h, int sec_w, cudaStream_t s) {
  if (T == 0) return 0;
  if (hd % 2 || 2 * half_rot > hd) return -2;
  if (pos_stride == 1 && 2 * half_rot == hd && hd % 16 == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    int thr = H * (hd / 16);
    thr = thr > 256 ? 256 : ((thr + 31) / 32) * 32;
    rope_full_vec_kernel<<<T, thr, hd * sizeof(float), s>>>((const bf16*)x, in_stride, (bf16*)out, out_stride, pos,
                                                            inv_freq, T, H, hd, inverse);
    CHECK_LAUNCH();
  }
  int threads = H * (hd / 2);
  threads = threads > 512 ? 512 : ((threads + 31) / 32) * 32;
  rope_kernel<<<T, threads, 0, s>>>((const bf16*)x, in_stride, (bf16*)out, out_stride, pos, inv_freq, T, H, hd,
                                    half_rot, inverse, pos_stride, sec_h, sec_w);
  CHECK_LAUNCH();
}

int ftb_glu_fwd(const void* gate, const void* up, void* out, long T, int F, int ld_in, int ld_out, int kind,
                cudaStream_t s) {
  if (T == 0) return 0;
  if (F % 8 || ld_in % 8 || ld_out % 8) return -2;
  const long nvec = T * (F / 8);
  const int blocks = (int)((nvec + 255) / 256 < 148 * 16 ? (nvec + 255) / 256 : 148 * 16);
  glu_fwd_kernel<<<blocks, 256, 0, s>>>((const bf16*)gate, (const bf16*)up, (bf16*)out, T, F, ld_in, ld_out, kind);
  CHECK_LAUNCH();
}
int ftb_glu_bwd(const void* dact, const void* gate, const void* up, void* dgate, void* dup, void* act_out, long T,
                int F, int ld_in, int ld_d, int ld_act, int kind, cudaStream_t s) {
  if (T == 0) return 0;
  if (F % 8 || ld_in % 8 || ld_d % 8 || ld_act % 8) return -2;
  const long nvec = T * (F / 8);
  const int blocks = (int)((nvec + 255) / 256 < 148 * 16 ? (nvec + 255) / 256 : 148 * 16);
  glu_bwd_kernel<<<blocks, 256, 0, s>>>((const bf16*)dact, (const bf16*)gate, (const bf16*)up, (bf16*)dgate,
                                        (bf16*)dup, (bf16*)act_out, T, F, ld_in, ld_d, ld_act, kind);
  CHECK_LAUNCH();
}

int ftb_glu_bwd_weighted(const void* dact, const void* gate, const void* up, const float* w_row, void* dgate, void* dup,
                         void* act_w, float* dw_row, long T, int F, int ld_in, int ld_d, int kind, cudaStream_t s) {
  if (T == 0) return 0;
  if (F % 8 || ld_in % 8 || ld_d % 8) return -2;
  glu_bwd_weighted_kernel<<<(unsigned)T, 128, 0, s>>>((const bf16*)dact, (const bf16*)gate, (const bf16*)up, w_row,
                                                      (bf16*)dgate, (bf16*)dup, (bf16*)act_w, dw_row, F, ld_in, ld_d, kind);
  CHECK_LAUNCH();
}

int ftb_softmax_ce(void* logits, const long* targets, const float* loss_mask, float* loss, int T, int V, long ld,
                   float grad_scale, float softcap, long ignore_index, cudaStream_t s) {
  if (T == 0) return 0;
  if (ld % 8) return -2;
  softmax_ce_kernel<<<T, CE_THREADS, 0, s>>>((bf16*)logits, targets, loss_mask, loss, T, V, ld, grad_scale, softcap,
                                             ignore_index);
  CHECK_LAUNCH();
}

int ftb_embedding_fwd(const long* tokens, const void* table, void* out, int T, int D, float scale, cudaStream_t s) {
  if (T == 0) return 0;
  if (D % 8) return -2;
  embedding_fwd_kernel<<<T, 128, 0, s>>>(tokens, (const bf16*)table, (bf16*)out, T, D, scale);
  CHECK_LAUNCH();
}
int ftb_embedding_bwd(const long* sorted_tok, const long* order, const void* dy, void* grad, int T, int D,
                      float scale, int grad_fp32, cudaStream_t s) {
  if (T == 0) return 0;
  if (D % 8) return -2;
  embedding_bwd_kernel<<<T, 128, 0, s>>>(sorted_tok, order, (const bf16*)dy, grad, T, D, scale, grad_fp32);
  CHECK_LAUNCH();
}

// Tensors are passed as parallel arrays (host memory) of length `count` <= 24.
int ftb_adamw_multi(int count, void** p, const void** g, void** m, void** v, const long* n, const float* lr,
                    const float* wd, const int* p_dt, const int* g_dt, const int* s_dt, float beta1, float beta2,
                    float eps, float bc1, float bc2, float grad_scale, cudaStream_t s) {
  if (count <= 0) return 0;
  if (count > ADAM_MAX) return -2;
  AdamArgs a;
  long blocks = 0;
  for (int i = 0; i < count; ++i) {
    a.t[i].p = p[i]; a.t[i].g = g[i]; a.t[i].m = m[i]; a.t[i].v = v[i];
    a.t[i].n = n[i]; a.t[i].block_start = blocks;
    a.t[i].lr = lr[i]; a.t[i].wd = wd[i];
    a.t[i].p_dt = p_dt[i]; a.t[i].g_dt = g_dt[i]; a.t[i].s_dt = s_dt[i]; a.t[i].pad = 0;
    blocks += (n[i] + ADAM_PER_BLOCK - 1) / ADAM_PER_BLOCK;
  }
  a.count = count; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.bc1 = bc1; a.bc2 = bc2; a.grad_scale = grad_scale;
  if (blocks == 0) return 0;
  adamw_kernel<<<(unsigned)blocks, ADAM_THREADS, 0, s>>>(a);
  CHECK_LAUNCH();
}

int ftb_gated_rmsnorm_fwd(const void* o, const void* z, const float* w, void* y, long rows, int D, float eps,
                          cudaStream_t s) {
  if (rows == 0) return 0;
  gated_rmsnorm_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const bf16*)o, (const bf16*)z, w, (bf16*)y,
                                                                       rows, D, eps);
  CHECK_LAUNCH();
}
int ftb_l2norm_fwd(const void* x, void* y, float* rnorm, long rows, int D, float eps, cudaStream_t s) {
  if (rows == 0) return 0;
  l2norm_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const bf16*)x, (bf16*)y, rnorm, rows, D, eps);
  CHECK_LAUNCH();
}

// Router backward (one warp per token, E <= 256): dlogits (T, E) fp32 from the gradient of the K routing weights.
//   mode 0 (softmax over the K picks):  dl[e_k] = w_k (dw_k - sum_j w_j dw_j), 0 elsewhere
//   mode 1 (softmax over E, then pick): dl = p * (dp - sum p dp) with dp = dw scattered to the picks
// (flextrain/ops/_kernels/moe.py:360-458).
__global__ void topk_route_bwd_kernel(const float* __restrict__ dw, const bf16* __restrict__ logits,
                                      const float* __restrict__ w, const int* __restrict__ experts,
                                      float* __restrict__ dl, int T, int E, int K, int mode) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  float* out = dl + (size_t)t * E;
  const float* dwt = dw + (size_t)t * K;
  const int* et = experts + (size_t)t * K;
  if (mode == 0) {
    const float* wt = w + (size_t)t * K;
    float dot = 0.f;
    for (int k = 0; k < K; ++k) dot += wt[k] * dwt[k];
    for (int e = lane; e < E; e += 32) out[e] = 0.f;
    __syncwarp();
    if (lane < K) out[et[lane]] = wt[lane] * (dwt[lane] - dot);
    return;
  }
  float v[8], dp[8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + j * 32;
    v[j] = e < E ? __bfloat162float(logits[(size_t)t * E + e]) : -INFINITY;
    dp[j] = 0.f;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { v[j] = (lane + j * 32 < E) ? __expf(v[j] - mx) : 0.f; sum += v[j]; }
  sum = warp_sum(sum);
  for (int k = 0; k < K; ++k) {
    const int e = et[k];
    if ((e & 31) == lane) dp[e >> 5] = dwt[k];
  }
  float dot = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { v[j] /= sum; dot += v[j] * dp[j]; }
  dot = warp_sum(dot);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + j * 32;
    if (e < E) out[e] = v[j] * (dp[j] - dot);
  }
}

// Load-balance auxiliary gradient added into dlogits (flextrain/ops/_kernels/moe.py:601-646):
//   dl[t, e] += alpha * p[t, e] * (gvec[e] - sum_j p[t, j] gvec[j]),  p = softmax(logits[t, :]),
//   gvec[e] = counts[e] / n_slots * E / total_tokens   (the routed fractions are constants of the step).
// One warp per token, E <= 256.
__global__ void load_balance_bwd_kernel(const bf16* __restrict__ logits, const int* __restrict__ counts,
                                        float* __restrict__ dl, int T, int E, float alpha, float gscale) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  float v[8], gv[8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + j * 32;
    v[j] = e < E ? __bfloat162float(logits[(size_t)t * E + e]) : -INFINITY;
    gv[j] = e < E ? (float)counts[e] * gscale : 0.f;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { v[j] = (lane + j * 32 < E) ? __expf(v[j] - mx) : 0.f; sum += v[j]; }
  sum = warp_sum(sum);
  float dot = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { v[j] /= sum; dot += v[j] * gv[j]; }
  dot = warp_sum(dot);
  float* out = dl + (size_t)t * E;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = lane + j * 32;
    if (e < E) out[e] += alpha * v[j] * (gv[j] - dot);
  }
}

int ftb_load_balance_bwd(const void* logits, const int* counts, float* dl, int T, int E, float alpha, float gscale,
                         cudaStream_t s) {
  if (T == 0) return 0;
  if (E > 256) return -2;
  load_balance_bwd_kernel<<<(T + 7) / 8, 256, 0, s>>>((const bf16*)logits, counts, dl, T, E, alpha, gscale);
  CHECK_LAUNCH();
}

int ftb_topk_route_bwd(const float* dw, const void* logits, const float* w, const int* experts, float* dl, int T, int E,
                       int K, int mode, cudaStream_t s) {
  if (T == 0) return 0;
  if (E > 256 || K > 32) return -2;
  topk_route_bwd_kernel<<<(T + 7) / 8, 256, 0, s>>>(dw, (const bf16*)logits, w, experts, dl, T, E, K, mode);
  CHECK_LAUNCH();
}

int ftb_topk_route(const void* logits, float* weights, int* experts, int T, int E, int K, int mode, cudaStream_t s) {
  if (T == 0) return 0;
  if (E > 256 || K > 16) return -2;
  topk_route_kernel<<<(T + 7) / 8, 256, 0, s>>>((const bf16*)logits, weights, experts, T, E, K, mode);
  CHECK_LAUNCH();
}
int ftb_gather_rows(const void* in, const int* idx, const float* w, void* out, long rows, int D, int idx_div,
                    cudaStream_t s) {
  if (rows == 0) return 0;
  if (D % 8) return -2;
  gather_rows_kernel<<<(unsigned)rows, 128, 0, s>>>((const bf16*)in, idx, w, (bf16*)out, rows, D, idx_div);
  CHECK_LAUNCH();
}
int ftb_moe_combine(const void* y, const int* inv, const float* w, const void* resid, void* out, int T, int K, int D,
                    cudaStream_t s) {
  if (T == 0) return 0;
  if (D % 8) return -2;
  moe_combine_kernel<<<T, 128, 0, s>>>((const bf16*)y, inv, w, (const bf16*)resid, (bf16*)out, T, K, D);
  CHECK_LAUNCH();
}

}  // extern "C"
