// Gated DeltaNet (gated delta rule) recurrence for sm_100a: forward and a hand-derived backward, token-recurrent.
//
// Per value head, with state S (dk x dv), log-decay g_t <= 0, write strength beta_t and unit-norm keys:
//     S^ = exp(g_t) S_{t-1};   r = S^^T k_t;   e = beta_t (v_t - r);   S_t = S^ + k_t e^T;   o_t = scale * S_t^T q_t
// The reference project calls FLA's chunked Triton kernels for this (flextrain/nn/blocks/linear_attn.py:1090-1145,
// 1702-1722).  Here the recurrence is run as written: the dv columns of S evolve independently, so a CTA owns a block
// of NC columns of one (sequence, head) and keeps its dk x NC slice of the state in registers for the whole
// sequence; sequences x heads x column blocks give thousands of CTAs for packed batches and HV * dv / NC CTAs for
// one long sequence.  No chunk-level triangular solves are needed.
//
// Thread layout (128 threads): ti = tid & 15 owns rows {ti + 16 rr}, tj = tid >> 4 owns columns {tj*CPT + cc}.
// Reductions over rows (r, o, de) are 4 xor-shuffles inside a half warp; reductions over columns (dq, dk) are
// accumulated per warp in shared memory over a block of TB tokens and flushed with fp32 atomics once per block.
//
// Backward (adjoint dS of the state, reverse in time), for dO_t given:
//     dS' = dS_t + scale q_t dO_t^T;  de = dS'^T k_t;  dv = beta de;  dbeta = de.(v - r);  dr = -beta de
//     dk_t = dS' e  +  S^ dr;         dq_t = scale S_t dO_t;          dS_{t-1} = exp(g_t) (dS' + k_t dr^T)
//     dg_t = sum_{u >= t} ( q_u.dq_u - k_u.(dS'_u e_u) + k_u.(S^_u dr_u) )  (+ <dS_final, S_final>)
// The terms that need the state itself (dq, S^ dr) are produced by re-running the forward recurrence ("pass F") with
// de from the reverse pass ("pass R").  Both passes add their part of the per-token scalar q.dq - k.(dS' e) + k.(S^ dr)
// into `sacc`; the caller turns it into dg with a suffix sum per sequence.  dq / dk are written per value head in fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

typedef __nv_bfloat16 bf16;
constexpr int TB = 8;            // tokens staged per block
constexpr int NT = 128;          // threads per CTA

struct GdnArgs {
  const bf16* q;       // (T, HK, DK)
  const bf16* k;       // (T, HK, DK)
  const bf16* v;       // (T, HV, DV)
  const float* g;      // (T, HV)
  const float* beta;   // (T, HV)
  const int* cu;       // (Nseq + 1)
  const float* state_in;   // (Nseq, HV, DK, DV) or null
  float* state_out;        // (Nseq, HV, DK, DV) or null   (forward: final state; pass R: gradient of the initial state)
  bf16* o;             // (T, HV, DV)        forward output
  float* r;            // (T, HV, DV)        forward: prediction S^^T k (kept for the backward) or null
  const bf16* d_o;     // (T, HV, DV)        backward
  float* de;           // (T, HV, DV)        pass R writes, pass F reads
  bf16* dv;            // (T, HV, DV)        pass R
  float* dbeta;        // (T, HV)            pass R (atomic over column blocks)
  float* dq;           // (T, HV, DK) fp32   pass F (atomic over column blocks)
  float* dk;           // (T, HV, DK) fp32   pass R adds dS' e, pass F adds S^ dr (atomic)
  float* sacc;         // (T, HV) fp32       per-token scalar of the gate gradient: q.dq - k.(dS' e) + k.(S^ dr)
  int HK, HV, DV;
  float scale;
};

__device__ __forceinline__ float half_warp_sum(float x) {   // over the 16 lanes that share tj
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

// Four per-column partial sums reduced over the 16 lanes of a half warp in 5 shuffles instead of 16: each exchange
// halves the number of columns a lane is responsible for (reduce-scatter), so after the xor-8 and xor-4 steps a lane
// carries one column, c = 2 * bit3(lane) + bit2(lane), and the xor-2 / xor-1 steps finish its sum.
__device__ __forceinline__ float reduce_scatter4(float p0, float p1, float p2, float p3, int lane) {
  const bool hi8 = lane & 8;
  float k0 = hi8 ? p2 : p0, k1 = hi8 ? p3 : p1;
  k0 += __shfl_xor_sync(0xffffffffu, hi8 ? p0 : p2, 8);
  k1 += __shfl_xor_sync(0xffffffffu, hi8 ? p1 : p3, 8);
  const bool hi4 = lane & 4;
  float k = hi4 ? k1 : k0;
  k += __shfl_xor_sync(0xffffffffu, hi4 ? k0 : k1, 4);
  k += __shfl_xor_sync(0xffffffffu, k, 2);
  k += __shfl_xor_sync(0xffffffffu, k, 1);
  return k;
}
// ... and handed back to every lane of the half warp (4 more shuffles).
__device__ __forceinline__ void all_gather4(float k, int lane, float (&out)[4]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) out[c] = __shfl_sync(0xffffffffu, k, (lane & 0x13) | (c << 2));
}

// Sum over the lanes that hold one token's DK consecutive elements (DK lanes for DK = 16, the whole warp otherwise).
template <int DK>
__device__ __forceinline__ float segment_sum(float x) {
  if (DK >= 32) x += __shfl_xor_sync(0xffffffffu, x, 16);
  return half_warp_sum(x);
}

// MODE 0: forward (o, r, final state).  MODE 1: pass F of the backward (dq, dk += S^ dr).
template <int RPT, int CPT, int MODE>
__global__ void __launch_bounds__(NT) gdn_forward_kernel(const GdnArgs a) {
  constexpr int DK = 16 * RPT, NC = 8 * CPT;
  __shared__ float k_s[TB][DK], q_s[TB][DK], v_s[TB][NC], x_s[TB][NC], y_s[TB][NC];
  __shared__ float a_s[TB], b_s[TB];
  __shared__ float acc_q[MODE == 1 ? 4 : 1][TB][MODE == 1 ? DK : 1];
  __shared__ float acc_k[MODE == 1 ? 4 : 1][TB][MODE == 1 ? DK : 1];
  const int tid = threadIdx.x, ti = tid & 15, tj = tid >> 4, warp = tid >> 5;
  const int col0 = blockIdx.x * NC, hv = blockIdx.y, seq = blockIdx.z;
  const int hk = hv / (a.HV / a.HK);
  const int t0 = a.cu[seq], t1 = a.cu[seq + 1];
  float S[RPT][CPT];
#pragma unroll
  for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
      const int i = ti + 16 * rr, j = col0 + tj * CPT + cc;
      S[rr][cc] = a.state_in ? a.state_in[(((size_t)seq * a.HV + hv) * DK + i) * a.DV + j] : 0.f;
    }
  for (int tb = t0; tb < t1; tb += TB) {
    const int nt = min(TB, t1 - tb);
    __syncthreads();
    for (int idx = tid; idx < nt * DK; idx += NT) {
      const int t = idx / DK, i = idx - t * DK;
      const size_t off = ((size_t)(tb + t) * a.HK + hk) * DK + i;
      k_s[t][i] = __bfloat162float(a.k[off]);
      q_s[t][i] = __bfloat162float(a.q[off]) * a.scale;
    }
    for (int idx = tid; idx < nt * NC; idx += NT) {
      const int t = idx / NC, j = idx - t * NC;
      const size_t off = ((size_t)(tb + t) * a.HV + hv) * a.DV + col0 + j;
      v_s[t][j] = __bfloat162float(a.v[off]);
      if (MODE == 1) {
        x_s[t][j] = __bfloat162float(a.d_o[off]);
        y_s[t][j] = a.de[off];
      }
    }
    if (tid < nt) {
      a_s[tid] = __expf(a.g[(size_t)(tb + tid) * a.HV + hv]);
      b_s[tid] = a.beta[(size_t)(tb + tid) * a.HV + hv];
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float at = a_s[t], bt = b_s[t];
      float kr[RPT], qr[RPT], rj[CPT];
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) { kr[rr] = k_s[t][ti + 16 * rr]; qr[rr] = q_s[t][ti + 16 * rr]; }
      {
        float pp[CPT];
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float p = 0.f;
#pragma unroll
          for (int rr = 0; rr < RPT; ++rr) { S[rr][cc] *= at; p += kr[rr] * S[rr][cc]; }
          pp[cc] = p;
        }
        if constexpr (CPT == 4) {
          all_gather4(reduce_scatter4(pp[0], pp[1], pp[2], pp[3], tid & 31), tid & 31, rj);
        } else {
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) rj[cc] = half_warp_sum(pp[cc]);
        }
      }
      if (MODE == 1) {   // dk += S^ dr  with dr = -beta de   (S holds S^ here)
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr) {
          float p = 0.f;
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) p += S[rr][cc] * (-bt * y_s[t][tj * CPT + cc]);
          p += __shfl_xor_sync(0xffffffffu, p, 16);
          if ((tid & 16) == 0) acc_k[warp][t][ti + 16 * rr] = p;
        }
      }
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const float e = bt * (v_s[t][tj * CPT + cc] - rj[cc]);
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr) S[rr][cc] += kr[rr] * e;
      }
      if (MODE == 0) {
        float pp[CPT];
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float p = 0.f;
#pragma unroll
          for (int rr = 0; rr < RPT; ++rr) p += qr[rr] * S[rr][cc];
          pp[cc] = p;
        }
        if constexpr (CPT == 4) {
          const float tot = reduce_scatter4(pp[0], pp[1], pp[2], pp[3], tid & 31);
          if ((ti & 3) == 0) {                     // lanes 0, 4, 8, 12 of the half warp hold columns 0..3
            const int cc = ti >> 2;
            const size_t off = ((size_t)(tb + t) * a.HV + hv) * a.DV + col0 + tj * CPT + cc;
            a.o[off] = __float2bfloat16(tot);
            if (a.r) a.r[off] = rj[cc];
          }
        } else {
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) {
            const float p = half_warp_sum(pp[cc]);
            if (ti == 0) {
              const size_t off = ((size_t)(tb + t) * a.HV + hv) * a.DV + col0 + tj * CPT + cc;
              a.o[off] = __float2bfloat16(p);
              if (a.r) a.r[off] = rj[cc];
            }
          }
        }
      } else {            // dq = scale S_t dO
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr) {
          float p = 0.f;
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) p += S[rr][cc] * x_s[t][tj * CPT + cc];
          p += __shfl_xor_sync(0xffffffffu, p, 16);
          if ((tid & 16) == 0) acc_q[warp][t][ti + 16 * rr] = p * a.scale;
        }
      }
    }
    if (MODE == 1) {
      __syncthreads();
      if (tid < TB) a_s[tid] = 0.f;           // reused as the per-token scalar accumulator of this block
      __syncthreads();
      for (int idx = tid; idx < TB * DK; idx += NT) {           // uniform trip count: the shuffles need full warps
        const int t = idx / DK, i = idx - t * DK;
        float sc = 0.f;
        if (t < nt) {
          const size_t off = ((size_t)(tb + t) * a.HV + hv) * DK + i;
          const float vq = acc_q[0][t][i] + acc_q[1][t][i] + acc_q[2][t][i] + acc_q[3][t][i];
          const float vk = acc_k[0][t][i] + acc_k[1][t][i] + acc_k[2][t][i] + acc_k[3][t][i];
          atomicAdd(a.dq + off, vq);
          atomicAdd(a.dk + off, vk);
          sc = q_s[t][i] * vq / a.scale + k_s[t][i] * vk;
        }
        sc = segment_sum<DK>(sc);
        if ((idx & (DK < 32 ? DK - 1 : 31)) == 0 && t < nt) atomicAdd(&a_s[t], sc);
      }
      __syncthreads();
      if (tid < nt) atomicAdd(a.sacc + (size_t)(tb + tid) * a.HV + hv, a_s[tid]);
    }
  }
  if (MODE == 0 && a.state_out) {
#pragma unroll
    for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const int i = ti + 16 * rr, j = col0 + tj * CPT + cc;
        a.state_out[(((size_t)seq * a.HV + hv) * DK + i) * a.DV + j] = S[rr][cc];
      }
  }
}

// Pass R: reverse in time.  state_in = gradient of the final state (or null), state_out = gradient of the initial one.
template <int RPT, int CPT>
__global__ void __launch_bounds__(NT) gdn_reverse_kernel(const GdnArgs a) {
  constexpr int DK = 16 * RPT, NC = 8 * CPT;
  __shared__ float k_s[TB][DK], q_s[TB][DK], v_s[TB][NC], x_s[TB][NC], r_s[TB][NC];
  __shared__ float a_s[TB], b_s[TB];
  __shared__ float acc_k[4][TB][DK];
  __shared__ float acc_b[4][TB];
  const int tid = threadIdx.x, ti = tid & 15, tj = tid >> 4, warp = tid >> 5;
  const int col0 = blockIdx.x * NC, hv = blockIdx.y, seq = blockIdx.z;
  const int hk = hv / (a.HV / a.HK);
  const int t0 = a.cu[seq], t1 = a.cu[seq + 1];
  float dS[RPT][CPT];
#pragma unroll
  for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
      const int i = ti + 16 * rr, j = col0 + tj * CPT + cc;
      dS[rr][cc] = a.state_in ? a.state_in[(((size_t)seq * a.HV + hv) * DK + i) * a.DV + j] : 0.f;
    }
  const int nblk = (t1 - t0 + TB - 1) / TB;
  for (int blk = nblk - 1; blk >= 0; --blk) {
    const int tb = t0 + blk * TB;
    const int nt = min(TB, t1 - tb);
    __syncthreads();
    for (int idx = tid; idx < nt * DK; idx += NT) {
      const int t = idx / DK, i = idx - t * DK;
      const size_t off = ((size_t)(tb + t) * a.HK + hk) * DK + i;
      k_s[t][i] = __bfloat162float(a.k[off]);
      q_s[t][i] = __bfloat162float(a.q[off]) * a.scale;
    }
    for (int idx = tid; idx < nt * NC; idx += NT) {
      const int t = idx / NC, j = idx - t * NC;
      const size_t off = ((size_t)(tb + t) * a.HV + hv) * a.DV + col0 + j;
      v_s[t][j] = __bfloat162float(a.v[off]);
      x_s[t][j] = __bfloat162float(a.d_o[off]);
      r_s[t][j] = a.r[off];
    }
    if (tid < nt) {
      a_s[tid] = __expf(a.g[(size_t)(tb + tid) * a.HV + hv]);
      b_s[tid] = a.beta[(size_t)(tb + tid) * a.HV + hv];
    }
    __syncthreads();
    for (int t = nt - 1; t >= 0; --t) {
      const float at = a_s[t], bt = b_s[t];
      float kr[RPT], qr[RPT], de[CPT], ej[CPT];
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) { kr[rr] = k_s[t][ti + 16 * rr]; qr[rr] = q_s[t][ti + 16 * rr]; }
      float db = 0.f;
      {
        float pp[CPT];
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          const float dO = x_s[t][tj * CPT + cc];
          float p = 0.f;
#pragma unroll
          for (int rr = 0; rr < RPT; ++rr) { dS[rr][cc] += qr[rr] * dO; p += kr[rr] * dS[rr][cc]; }
          pp[cc] = p;
        }
        if constexpr (CPT == 4) {
          all_gather4(reduce_scatter4(pp[0], pp[1], pp[2], pp[3], tid & 31), tid & 31, de);
        } else {
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) de[cc] = half_warp_sum(pp[cc]);
        }
      }
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const float diff = v_s[t][tj * CPT + cc] - r_s[t][tj * CPT + cc];
        ej[cc] = bt * diff;
        db += de[cc] * diff;
        if (ti == 0) {
          const size_t off = ((size_t)(tb + t) * a.HV + hv) * a.DV + col0 + tj * CPT + cc;
          a.de[off] = de[cc];
          a.dv[off] = __float2bfloat16(bt * de[cc]);
        }
      }
      db += __shfl_xor_sync(0xffffffffu, db, 16);       // every lane of a half warp holds the same db
      if ((tid & 31) == 0) acc_b[warp][t] = db;
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) {
        float p = 0.f;
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) p += dS[rr][cc] * ej[cc];
        p += __shfl_xor_sync(0xffffffffu, p, 16);
        if ((tid & 16) == 0) acc_k[warp][t][ti + 16 * rr] = p;
      }
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const float dr = -bt * de[cc];
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr) dS[rr][cc] = at * (dS[rr][cc] + kr[rr] * dr);
      }
    }
    __syncthreads();
    if (tid < TB) a_s[tid] = 0.f;             // reused as the per-token scalar accumulator of this block
    __syncthreads();
    for (int idx = tid; idx < TB * DK; idx += NT) {             // uniform trip count: the shuffles need full warps
      const int t = idx / DK, i = idx - t * DK;
      float sc = 0.f;
      if (t < nt) {
        const float vk = acc_k[0][t][i] + acc_k[1][t][i] + acc_k[2][t][i] + acc_k[3][t][i];
        atomicAdd(a.dk + ((size_t)(tb + t) * a.HV + hv) * DK + i, vk);
        sc = -k_s[t][i] * vk;
      }
      sc = segment_sum<DK>(sc);
      if ((idx & (DK < 32 ? DK - 1 : 31)) == 0 && t < nt) atomicAdd(&a_s[t], sc);
    }
    __syncthreads();
    if (tid < nt) {
      atomicAdd(a.dbeta + (size_t)(tb + tid) * a.HV + hv, acc_b[0][tid] + acc_b[1][tid] + acc_b[2][tid] + acc_b[3][tid]);
      atomicAdd(a.sacc + (size_t)(tb + tid) * a.HV + hv, a_s[tid]);
    }
  }
  if (a.state_out) {
#pragma unroll
    for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const int i = ti + 16 * rr, j = col0 + tj * CPT + cc;
        a.state_out[(((size_t)seq * a.HV + hv) * DK + i) * a.DV + j] = dS[rr][cc];
      }
  }
}

template <int RPT, int CPT>
int launch_all(int pass, const GdnArgs& a, int nseq, cudaStream_t s) {
  dim3 grid(a.DV / (8 * CPT), a.HV, nseq);
  if (pass == 0) gdn_forward_kernel<RPT, CPT, 0><<<grid, NT, 0, s>>>(a);
  else if (pass == 1) gdn_reverse_kernel<RPT, CPT><<<grid, NT, 0, s>>>(a);
  else gdn_forward_kernel<RPT, CPT, 1><<<grid, NT, 0, s>>>(a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -400 - (int)e;
}

// Column block per CTA: 32 columns when that already gives two CTAs per SM, otherwise 16 or 8 so that one long
// sequence still spreads over the whole GPU (the recurrence is latency-bound per CTA).
int cols_per_thread(int nseq, int HV, int DV) {
  const long heads = (long)nseq * HV;
  if (DV % 32 == 0 && heads * (DV / 32) >= 296) return 4;
  if (DV % 16 == 0 && heads * (DV / 16) >= 296) return 2;
  if (DV % 8 == 0) return 1;
  return 0;
}

template <int RPT>
int launch_cols(int pass, const GdnArgs& a, int nseq, cudaStream_t s) {
  switch (cols_per_thread(nseq, a.HV, a.DV)) {
    case 4: return launch_all<RPT, 4>(pass, a, nseq, s);
    case 2: return launch_all<RPT, 2>(pass, a, nseq, s);
    case 1: return launch_all<RPT, 1>(pass, a, nseq, s);
    default: return -2;
  }
}

}  // namespace

extern "C" {

// pass: 0 forward, 1 backward reverse pass, 2 backward forward-direction pass.  DK in {16, 32, 64, 128}, DV % 8 == 0.
// Number of column blocks (CTAs per head) the kernels will use: the leading dimension of the dq / dk partial buffers.
int ftb_gdn_col_blocks(int nseq, int HV, int DV) {
  const int cpt = cols_per_thread(nseq, HV, DV);
  return cpt ? DV / (8 * cpt) : 0;
}

int ftb_gdn(int pass, const void* q, const void* k, const void* v, const float* g, const float* beta, const int* cu,
            int nseq, const float* state_in, float* state_out, void* o, float* r, const void* d_o, float* de, void* dv,
            float* dbeta, float* dq, float* dk, float* sacc, int HK, int HV, int DK, int DV, float scale,
            cudaStream_t s) {
  if (nseq <= 0) return 0;
  if (HV % HK) return -2;
  GdnArgs a;
  a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.g = g; a.beta = beta; a.cu = cu;
  a.state_in = state_in; a.state_out = state_out; a.o = (bf16*)o; a.r = r; a.d_o = (const bf16*)d_o; a.de = de;
  a.dv = (bf16*)dv; a.dbeta = dbeta; a.dq = dq; a.dk = dk; a.sacc = sacc; a.HK = HK; a.HV = HV; a.DV = DV; a.scale = scale;
  switch (DK) {
    case 16: return launch_cols<1>(pass, a, nseq, s);
    case 32: return launch_cols<2>(pass, a, nseq, s);
    case 64: return launch_cols<4>(pass, a, nseq, s);
    case 128: return launch_cols<8>(pass, a, nseq, s);
    default: return -2;
  }
}

}  // extern "C"
