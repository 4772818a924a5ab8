// Peer-memory communication kernels for one NVSwitch box (one process per GPU).
//
// The reference project has no collective at all (single GPU).  These kernels are the data-parallel
// hot path of this framework; none of them calls NCCL.  Every rank maps every peer's buffers
// (CUDA IPC) and the kernels load / store peer memory directly over NVLink:
//
//   ftb_comm_signal_wait      per-(slot) flag exchange: "my data for `slot` is final" is stored into every
//                             peer's flag table, then the kernel waits (bounded) for all peers' flags.
//   ftb_comm_reduce_scatter   fused gradient reduce-scatter + bf16->fp32 cast + 1/tokens scale: each rank
//                             sums ITS element range of all ranks' gradient buffers into a local fp32 shard.
//   ftb_comm_adamw_push       fused sharded AdamW + parameter all-gather: the owner updates its range in
//                             fp32 registers and stores the new bf16 values into every rank's parameter
//                             buffer (the all-gather is the store loop of the optimizer).
//   ftb_comm_allgather_push / ftb_comm_gather_rows_pull   building blocks for TP / EP paths.
//
// Waits are bounded by wall-clock (globaltimer): on expiry the kernel records an error word and
// returns, so a missing peer can never hang the GPU.  No TMA multicast and no multimem is used here.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;
constexpr int MAX_RANKS = 8;
constexpr int MAX_SEGS = 16;

static __device__ int g_error_word = 0;
static __device__ int g_error_where = 0;
__device__ __forceinline__ void set_error(int code, int where) {
  if (atomicCAS(&g_error_word, 0, code) == 0) g_error_where = where;
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerTable {
  void* ptr[MAX_RANKS];
};

// flags layout on every rank: int flags[num_slots][MAX_RANKS]; flags[slot][src] is written by rank `src`.
__global__ void signal_wait_kernel(PeerTable flag_tables, int slot, int rank, int world, int epoch,
                                   unsigned long long timeout_ns, int* status) {
  const int t = threadIdx.x;
  __threadfence_system();  // everything this stream wrote before is visible before the flag
  if (t < world) {
    int* peer_flags = reinterpret_cast<int*>(flag_tables.ptr[t]) + (size_t)slot * MAX_RANKS + rank;
    st_release_sys(peer_flags, epoch);
  }
  if (t < world) {
    const int* mine = reinterpret_cast<const int*>(flag_tables.ptr[rank]) + (size_t)slot * MAX_RANKS + t;
    const unsigned long long t0 = globaltimer_ns();
    bool ok = false;
    while (true) {
      if (ld_acquire_sys(mine) >= epoch) { ok = true; break; }
      if (globaltimer_ns() - t0 > timeout_ns) break;
      __nanosleep(200);
    }
    if (!ok) {
      set_error(2, slot * 100 + t);
      if (status) atomicExch(status, 1 + t);
    }
  }
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

// One segment = a run of same-dtype elements inside the (identically laid out) per-rank buffers.
struct Seg {
  long byte_off;     // offset of the segment inside each rank's buffer
  long begin;        // first element of this rank's range inside the segment
  long count;        // elements in this rank's range
  long out_off;      // element offset in the local shard arrays (fp32 grad / m / v)
  int dtype;         // 0 bf16, 1 fp32
  int pad;
};
struct SegTable {
  Seg s[MAX_SEGS];
  long block_start[MAX_SEGS + 1];
  int n;
};
constexpr int RS_THREADS = 256;
constexpr int RS_PER_BLOCK = RS_THREADS * 8;

__device__ __forceinline__ int find_seg(const SegTable& t, long block) {
  int k = 0;
#pragma unroll 1
  for (int i = 1; i < t.n; ++i)
    if (block >= t.block_start[i]) k = i;
  return k;
}

// out[out_off + i] = scale * sum_r buf_r[byte_off][begin + i]
__global__ void __launch_bounds__(RS_THREADS) reduce_scatter_kernel(PeerTable bufs, const __grid_constant__ SegTable tab,
                                                                     float* __restrict__ out, int world, int rank,
                                                                     float scale) {
  const int k = find_seg(tab, blockIdx.x);
  const Seg& sg = tab.s[k];
  const long base = ((long)blockIdx.x - tab.block_start[k]) * RS_PER_BLOCK;
  if (sg.dtype == 0) {
    const long i0 = base + (long)threadIdx.x * 8;
    if (i0 >= sg.count) return;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (i0 + 8 <= sg.count && ((sg.begin + i0) & 7) == 0) {
      for (int rr = 0; rr < world; ++rr) {
        const int r = (rank + rr) % world;   // start with the local copy, stagger the peers
        const bf16* src = reinterpret_cast<const bf16*>(reinterpret_cast<const char*>(bufs.ptr[r]) + sg.byte_off);
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(src + sg.begin + i0), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
      float4* o = reinterpret_cast<float4*>(out + sg.out_off + i0);
      o[0] = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
      o[1] = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
    } else {
      for (int e = 0; e < 8 && i0 + e < sg.count; ++e) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) {
          const bf16* src = reinterpret_cast<const bf16*>(reinterpret_cast<const char*>(bufs.ptr[r]) + sg.byte_off);
          a += __bfloat162float(src[sg.begin + i0 + e]);
        }
        out[sg.out_off + i0 + e] = a * scale;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long i = base + threadIdx.x + (long)j * RS_THREADS;
      if (i < sg.count) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) {
          const float* src = reinterpret_cast<const float*>(reinterpret_cast<const char*>(bufs.ptr[r]) + sg.byte_off);
          a += src[sg.begin + i];
        }
        out[sg.out_off + i] = a * scale;
      }
    }
  }
}

// The same reduce-scatter through the NVSwitch: `mc` is the multicast address of the symmetric gradient arena (every
// rank's copy bound to one multicast object), so ONE `multimem.ld_reduce` returns the sum over all ranks, added inside
// the switch with fp32 accumulation: this rank pulls count elements instead of world x count, and no SM adds anything.
// bf16 segments come back as bf16 (the switch rounds the fp32 sum once), fp32 segments as fp32.  Ranges that are not
// 16-byte aligned (never the case for ranges cut by shard_range) fall back to the peer-pointer loop.
__global__ void __launch_bounds__(RS_THREADS) reduce_scatter_mc_kernel(const char* __restrict__ mc, PeerTable bufs,
                                                                        const __grid_constant__ SegTable tab,
                                                                        float* __restrict__ out, int world, float scale) {
  const int k = find_seg(tab, blockIdx.x);
  const Seg& sg = tab.s[k];
  const long base = ((long)blockIdx.x - tab.block_start[k]) * RS_PER_BLOCK;
  if (sg.dtype == 0) {
    const long i0 = base + (long)threadIdx.x * 8;
    if (i0 >= sg.count) return;
    if (i0 + 8 <= sg.count && ((sg.begin + i0) & 7) == 0 && (sg.byte_off & 15) == 0) {
      const char* a = mc + sg.byte_off + (sg.begin + i0) * 2;
      uint4 u;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                   : "l"(a)
                   : "memory");
      float f[8];
      unpack8(u, f);
      float4* o = reinterpret_cast<float4*>(out + sg.out_off + i0);
      o[0] = make_float4(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
      o[1] = make_float4(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
    } else {
      for (int e = 0; e < 8 && i0 + e < sg.count; ++e) {
        float acc = 0.f;
        for (int r = 0; r < world; ++r) {
          const bf16* src = reinterpret_cast<const bf16*>(reinterpret_cast<const char*>(bufs.ptr[r]) + sg.byte_off);
          acc += __bfloat162float(src[sg.begin + i0 + e]);
        }
        out[sg.out_off + i0 + e] = acc * scale;
      }
    }
  } else {
    // fp32 segments (norm gains): four elements per 16-byte in-switch reduction
    const long i0 = base + (long)threadIdx.x * 8;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long i = i0 + 4 * h;
      if (i >= sg.count) break;
      if (i + 4 <= sg.count && ((sg.begin + i) & 3) == 0 && (sg.byte_off & 15) == 0) {
        const char* a = mc + sg.byte_off + (sg.begin + i) * 4;
        float4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                     : "l"(a)
                     : "memory");
        *reinterpret_cast<float4*>(out + sg.out_off + i) = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
      } else {
        for (int e = 0; e < 4 && i + e < sg.count; ++e) {
          float acc = 0.f;
          for (int r = 0; r < world; ++r) {
            const float* src = reinterpret_cast<const float*>(reinterpret_cast<const char*>(bufs.ptr[r]) + sg.byte_off);
            acc += src[sg.begin + i + e];
          }
          out[sg.out_off + i + e] = acc * scale;
        }
      }
    }
  }
}

struct AdamHyper {
  float lr, beta1, beta2, eps, wd, bc1, bc2;
};

// Owner update of this rank's range + store of the new parameter values into every rank's buffer.
// wd_mask bit k: apply weight decay to segment k.  State arrays m, v are fp32 shards (same indexing as grad).
__global__ void __launch_bounds__(RS_THREADS) adamw_push_kernel(PeerTable params, const __grid_constant__ SegTable tab,
                                                                 const float* __restrict__ grad, float* __restrict__ m,
                                                                 float* __restrict__ v, int world, int rank,
                                                                 AdamHyper h, unsigned wd_mask) {
  const int k = find_seg(tab, blockIdx.x);
  const Seg& sg = tab.s[k];
  const long base = ((long)blockIdx.x - tab.block_start[k]) * RS_PER_BLOCK;
  const float wd = ((wd_mask >> k) & 1u) ? h.wd : 0.f;
  if (sg.dtype == 0) {
    const long i0 = base + (long)threadIdx.x * 8;
    if (i0 >= sg.count) return;
    const bool vec = (i0 + 8 <= sg.count) && (((sg.begin + i0) & 7) == 0);
    const int n = vec ? 8 : (int)min((long)8, sg.count - i0);
    bf16* mine = reinterpret_cast<bf16*>(reinterpret_cast<char*>(params.ptr[rank]) + sg.byte_off) + sg.begin + i0;
    float p[8];
    if (vec) unpack8(*reinterpret_cast<const uint4*>(mine), p);
    else for (int e = 0; e < n; ++e) p[e] = __bfloat162float(mine[e]);
    const long s0 = sg.out_off + i0;
    if (vec && ((s0 & 3) == 0)) {
      // 16-byte accesses to the fp32 shard arrays: a lane-per-8-elements layout read with scalar loads touches every
      // 32-byte sector eight times
      float g8[8], m8[8], v8[8];
      *reinterpret_cast<float4*>(g8) = *reinterpret_cast<const float4*>(grad + s0);
      *reinterpret_cast<float4*>(g8 + 4) = *reinterpret_cast<const float4*>(grad + s0 + 4);
      *reinterpret_cast<float4*>(m8) = *reinterpret_cast<const float4*>(m + s0);
      *reinterpret_cast<float4*>(m8 + 4) = *reinterpret_cast<const float4*>(m + s0 + 4);
      *reinterpret_cast<float4*>(v8) = *reinterpret_cast<const float4*>(v + s0);
      *reinterpret_cast<float4*>(v8 + 4) = *reinterpret_cast<const float4*>(v + s0 + 4);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        p[e] -= h.lr * wd * p[e];
        m8[e] = h.beta1 * m8[e] + (1.f - h.beta1) * g8[e];
        v8[e] = h.beta2 * v8[e] + (1.f - h.beta2) * g8[e] * g8[e];
        p[e] -= h.lr * (m8[e] / h.bc1) / (sqrtf(v8[e] / h.bc2) + h.eps);
      }
      *reinterpret_cast<float4*>(m + s0) = *reinterpret_cast<const float4*>(m8);
      *reinterpret_cast<float4*>(m + s0 + 4) = *reinterpret_cast<const float4*>(m8 + 4);
      *reinterpret_cast<float4*>(v + s0) = *reinterpret_cast<const float4*>(v8);
      *reinterpret_cast<float4*>(v + s0 + 4) = *reinterpret_cast<const float4*>(v8 + 4);
    } else {
      for (int e = 0; e < n; ++e) {
        const long si = s0 + e;
        const float g = grad[si];
        float mm = m[si], vv = v[si];
        p[e] -= h.lr * wd * p[e];
        mm = h.beta1 * mm + (1.f - h.beta1) * g;
        vv = h.beta2 * vv + (1.f - h.beta2) * g * g;
        p[e] -= h.lr * (mm / h.bc1) / (sqrtf(vv / h.bc2) + h.eps);
        m[si] = mm;
        v[si] = vv;
      }
    }
    if (vec) {
      const uint4 packed = pack8(p);
      for (int rr = 0; rr < world; ++rr) {
        const int r = (rank + rr) % world;
        bf16* dst = reinterpret_cast<bf16*>(reinterpret_cast<char*>(params.ptr[r]) + sg.byte_off) + sg.begin + i0;
        *reinterpret_cast<uint4*>(dst) = packed;
      }
    } else {
      for (int r = 0; r < world; ++r) {
        bf16* dst = reinterpret_cast<bf16*>(reinterpret_cast<char*>(params.ptr[r]) + sg.byte_off) + sg.begin + i0;
        for (int e = 0; e < n; ++e) dst[e] = __float2bfloat16(p[e]);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long i = base + threadIdx.x + (long)j * RS_THREADS;
      if (i < sg.count) {
        const long si = sg.out_off + i;
        float* mine = reinterpret_cast<float*>(reinterpret_cast<char*>(params.ptr[rank]) + sg.byte_off) + sg.begin + i;
        float p = *mine;
        const float g = grad[si];
        float mm = m[si], vv = v[si];
        p -= h.lr * wd * p;
        mm = h.beta1 * mm + (1.f - h.beta1) * g;
        vv = h.beta2 * vv + (1.f - h.beta2) * g * g;
        p -= h.lr * (mm / h.bc1) / (sqrtf(vv / h.bc2) + h.eps);
        m[si] = mm;
        v[si] = vv;
        for (int r = 0; r < world; ++r)
          reinterpret_cast<float*>(reinterpret_cast<char*>(params.ptr[r]) + sg.byte_off)[sg.begin + i] = p;
      }
    }
  }
}

// Push a contiguous byte range of the local buffer to the same offset of every peer (all-gather by stores).
__global__ void allgather_push_kernel(PeerTable bufs, long byte_off, long nbytes, int world, int rank) {
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(bufs.ptr[rank]) + byte_off);
  const long n16 = nbytes >> 4;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int rr = 1; rr < world; ++rr) {
      const int r = (rank + rr) % world;
      reinterpret_cast<uint4*>(reinterpret_cast<char*>(bufs.ptr[r]) + byte_off)[i] = v;
    }
  }
}

// Pull rows from peers: out[i, :] = peer[src_rank[i]].base[src_row[i], :]  (bf16 rows of D elements).
// Used by expert-parallel dispatch (tokens pulled into expert-major order) and combine.
__global__ void gather_rows_pull_kernel(PeerTable bufs, const int* __restrict__ src_rank, const int* __restrict__ src_row,
                                        bf16* __restrict__ out, long rows, int D, long byte_off) {
  const long r = blockIdx.x;
  if (r >= rows) return;
  const int pr = src_rank[r];
  uint4* dst = reinterpret_cast<uint4*>(out + r * D);
  if (pr < 0) {
    for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(
                         reinterpret_cast<const char*>(bufs.ptr[pr]) + byte_off) + (long)src_row[r] * D);
  for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) dst[c] = src[c];
}

// out[i] = sum_r slots[r * slot_stride + i] (+ resid[i]); bf16 in / out, fp32 sum.  The tail of the GEMM -> reduce-scatter
// path: `slots` is this rank's staging area holding one partial panel per source rank.
__global__ void reduce_slots_kernel(const bf16* __restrict__ slots, long slot_stride, int world,
                                    const bf16* __restrict__ resid, bf16* __restrict__ out, long n) {
  const long n8 = n >> 3;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (resid) unpack8(reinterpret_cast<const uint4*>(resid)[i], acc);
    for (int r = 0; r < world; ++r) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(slots + (size_t)r * slot_stride)[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(acc);
  }
}

}  // namespace

static int fill_table(SegTable& t, int n, const long* byte_off, const long* begin, const long* count,
                      const long* out_off, const int* dtype, long* total_blocks) {
  if (n > MAX_SEGS) return -2;
  long blocks = 0;
  for (int i = 0; i < n; ++i) {
    t.s[i].byte_off = byte_off[i]; t.s[i].begin = begin[i]; t.s[i].count = count[i];
    t.s[i].out_off = out_off[i]; t.s[i].dtype = dtype[i]; t.s[i].pad = 0;
    t.block_start[i] = blocks;
    blocks += (count[i] + RS_PER_BLOCK - 1) / RS_PER_BLOCK;
  }
  t.block_start[n] = blocks;
  t.n = n;
  *total_blocks = blocks;
  return 0;
}

#define CHECK_LAUNCH()                                 \
  do {                                                 \
    cudaError_t e_ = cudaGetLastError();               \
    return e_ == cudaSuccess ? 0 : -400 - (int)e_;     \
  } while (0)

extern "C" {

// ---- symmetric heap plumbing (CUDA IPC). Handles are 64 opaque bytes exchanged through torch.distributed.
int ftb_comm_alloc(void** out, size_t nbytes) {
  cudaError_t e = cudaMalloc(out, nbytes);
  if (e != cudaSuccess) return -(int)e;
  e = cudaMemset(*out, 0, nbytes);
  return e == cudaSuccess ? 0 : -(int)e;
}
int ftb_comm_free(void* p) { return -(int)cudaFree(p); }
int ftb_comm_ipc_get(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return -(int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
int ftb_comm_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -(int)e;
}
int ftb_comm_ipc_close(void* p) { return -(int)cudaIpcCloseMemHandle(p); }

int ftb_comm_signal_wait(void* const* flag_tables, int slot, int rank, int world, int epoch, double timeout_s,
                         int* status, cudaStream_t s) {
  if (world > MAX_RANKS) return -2;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.ptr[i] = flag_tables[i];
  signal_wait_kernel<<<1, 32, 0, s>>>(t, slot, rank, world, epoch, (unsigned long long)(timeout_s * 1e9), status);
  CHECK_LAUNCH();
}

int ftb_comm_reduce_scatter(void* const* bufs, int n, const long* byte_off, const long* begin, const long* count,
                            const long* out_off, const int* dtype, float* out, int world, int rank, float scale,
                            cudaStream_t s) {
  if (world > MAX_RANKS) return -2;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.ptr[i] = bufs[i];
  SegTable tab;
  long blocks = 0;
  int rc = fill_table(tab, n, byte_off, begin, count, out_off, dtype, &blocks);
  if (rc) return rc;
  if (blocks == 0) return 0;
  reduce_scatter_kernel<<<(unsigned)blocks, RS_THREADS, 0, s>>>(t, tab, out, world, rank, scale);
  CHECK_LAUNCH();
}

// `mc` = multicast address of the same symmetric buffer (see reduce_scatter_mc_kernel); `bufs` are the peer mappings
// used for ranges that are not 16-byte aligned.
int ftb_comm_reduce_scatter_mc(const void* mc, void* const* bufs, int n, const long* byte_off, const long* begin,
                               const long* count, const long* out_off, const int* dtype, float* out, int world,
                               float scale, cudaStream_t s) {
  if (world > MAX_RANKS || mc == nullptr) return -2;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.ptr[i] = bufs[i];
  SegTable tab;
  long blocks = 0;
  int rc = fill_table(tab, n, byte_off, begin, count, out_off, dtype, &blocks);
  if (rc) return rc;
  if (blocks == 0) return 0;
  reduce_scatter_mc_kernel<<<(unsigned)blocks, RS_THREADS, 0, s>>>(reinterpret_cast<const char*>(mc), t, tab, out, world,
                                                                   scale);
  CHECK_LAUNCH();
}

int ftb_comm_adamw_push(void* const* params, int n, const long* byte_off, const long* begin, const long* count,
                        const long* out_off, const int* dtype, const float* grad, float* m, float* v, int world,
                        int rank, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                        unsigned wd_mask, cudaStream_t s) {
  if (world > MAX_RANKS) return -2;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.ptr[i] = params[i];
  SegTable tab;
  long blocks = 0;
  int rc = fill_table(tab, n, byte_off, begin, count, out_off, dtype, &blocks);
  if (rc) return rc;
  if (blocks == 0) return 0;
  AdamHyper h{lr, beta1, beta2, eps, wd, bc1, bc2};
  adamw_push_kernel<<<(unsigned)blocks, RS_THREADS, 0, s>>>(t, tab, grad, m, v, world, rank, h, wd_mask);
  CHECK_LAUNCH();
}

int ftb_comm_allgather_push(void* const* bufs, long byte_off, long nbytes, int world, int rank, cudaStream_t s) {
  if (world > MAX_RANKS || (nbytes & 15) || (byte_off & 15)) return -2;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.ptr[i] = bufs[i];
  if (nbytes == 0) return 0;
  long blocks = (nbytes / 16 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  allgather_push_kernel<<<(unsigned)blocks, 256, 0, s>>>(t, byte_off, nbytes, world, rank);
  CHECK_LAUNCH();
}

int ftb_comm_gather_rows_pull(void* const* bufs, const int* src_rank, const int* src_row, void* out, long rows, int D,
                              long byte_off, int world, cudaStream_t s) {
  if (world > MAX_RANKS || (D & 7)) return -2;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.ptr[i] = bufs[i];
  if (rows == 0) return 0;
  gather_rows_pull_kernel<<<(unsigned)rows, 128, 0, s>>>(t, src_rank, src_row, (bf16*)out, rows, D, byte_off);
  CHECK_LAUNCH();
}

int ftb_comm_reduce_slots(const void* slots, long slot_stride, int world, const void* resid, void* out, long n,
                          cudaStream_t s) {
  if (n == 0) return 0;
  if ((n & 7) || (slot_stride & 7)) return -2;
  long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  reduce_slots_kernel<<<(unsigned)blocks, 256, 0, s>>>((const bf16*)slots, slot_stride, world, (const bf16*)resid,
                                                       (bf16*)out, n);
  CHECK_LAUNCH();
}

int ftb_comm_error(void) {
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
