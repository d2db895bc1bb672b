// Peer-memory collectives over NVLink / NVSwitch, issued from inside kernels.
//
// Every rank owns one "symmetric" allocation of identical layout (a flag area
// followed by data).  Ranks exchange CUDA IPC handles once and map each other's
// allocation; after that a kernel reaches any peer with plain loads and stores.
//
//   gb_comm_fused_step   reduce-scatter of a gradient bucket in fixed rank
//                        order -> 1/W scale -> (a) write the mean to every
//                        rank (all-reduce-mean) or (b) AdamW on the owned 1/W
//                        shard (fp32 master, m, v) and write the updated 16-bit
//                        parameters to every rank (ZeRO-1 step): one kernel does
//                        the collective and the math.
//   gb_comm_allreduce_small  one-shot sum of a short fp32 vector
//   gb_comm_broadcast    root's data region -> every rank
//   gb_comm_barrier      flag barrier
//
// The reference's collectives are a TCP star through rank 0 with a
// deterministic rank-order sum and identical bytes on every rank
// (distributed/distributed.go:249-416); DDPStep is all-reduce then step
// (:422-428).  Here each slice of a bucket is reduced by exactly one rank, in
// rank order, and that rank's result is what every rank receives, so the
// "identical bytes everywhere, run to run" contract still holds.
//
// Synchronisation uses epoch-numbered flags (never reset): CTA b of rank r
// writes epoch e into slot [b][r] of every peer's flag area and waits until its
// own slots [b][*] hold e.  Waits are bounded; on expiry the kernel records
// ST_COMM_TIMEOUT in the status word and returns.
//
// A test on one GPU can run all W ranks inside ONE cooperative launch
// (gridDim.y = W emulated ranks): separate launches that wait on each other are
// never used on a single device.
#include <string.h>

#include "comm_dev.cuh"

using namespace gb;
using namespace gbc;

namespace {

struct Comm {
  int rank = 0, world = 1;
  void* local = nullptr;
  size_t bytes = 0;
  PeerTable peers;
  void* mc_base = nullptr;   // multicast alias of the symmetric buffers (NVSwitch), or null
  bool attached = false;     // buffers mapped by the caller (gb_comm_attach): nothing to free here
  bool opened[kMaxWorld] = {false};
  unsigned int epoch = 0;
  unsigned int serial = 0;
  // capture mode (see comm_dev.cuh): device words holding the bases, and relative counters
  unsigned int* cap_bases = nullptr;  // [0] epoch base, [1] serial base
  unsigned int cap_epochs = 0, cap_serials = 0;
};

Comm g_comm;
int g_use_multimem = 1;   // used whenever a multicast mapping is attached; gb_comm_multimem(0) turns it off


struct StepArgs {
  PeerTable pt;
  int rank, world;
  int emulate;               // 1: gridDim.y emulated ranks inside one launch (single-GPU tests)
  long long grad_off;        // byte offset of the bucket's gradients inside the symmetric buffer
  long long param_off;       // byte offset of the bucket's parameters (mode 1)
  long long n;               // elements in the bucket (multiple of world * 8)
  int mode;                  // 0: all-reduce-mean into the gradients; 1: sharded AdamW + all-gather
  int dtype_bf16;            // element type: 0 fp16, 1 bf16, 2 fp32 (mode 0 only)
  int interleave;            // work mapping of the CTAs (see the kernel)
  unsigned int epoch;        // barrier epochs epoch (start) and epoch+1 (end)
  const unsigned int* epoch_base;  // added to `epoch` at run time when not null (graph replay)
  void* mc;                  // multicast alias of the buffers: reductions and broadcasts go through NVSwitch
  const float* hyper_dev;    // when not null: lr .. gscale are read from these 8 floats at run time
  float* master[kMaxWorld];  // per emulated rank (index 0 in real runs): fp32 shard state
  float* m[kMaxWorld];
  float* v[kMaxWorld];
  int opt_kind;              // mode 1: 0 AdamW, 1 SGD with momentum (coupled decay), 2 Lion
  int phase;                 // mode 1: 0 whole step; 1 reduce-scatter into gshard + sum of squares; 2 update from gshard + all-gather
  const unsigned char* wd_mask[kMaxWorld];  // one byte per 8 elements of the shard: 0 = no weight decay (null: all decay)
  float* gshard[kMaxWorld];  // phases 1 / 2: the averaged gradient shard in fp32
  float* sqpart[kMaxWorld];  // phase 1: per-CTA sums of squares of the averaged shard, [gridDim.x]
  float lr, wd, b1, b2, eps, bc1, bc2, gscale;
  int* status;
};

__device__ __forceinline__ void unpack8(const uint4& u, float* f, int bf) {
  float2 a;
  a = bf ? unpack_bf16(u.x) : unpack_f16(u.x); f[0] = a.x; f[1] = a.y;
  a = bf ? unpack_bf16(u.y) : unpack_f16(u.y); f[2] = a.x; f[3] = a.y;
  a = bf ? unpack_bf16(u.z) : unpack_f16(u.z); f[4] = a.x; f[5] = a.y;
  a = bf ? unpack_bf16(u.w) : unpack_f16(u.w); f[6] = a.x; f[7] = a.y;
}
__device__ __forceinline__ uint4 pack8(const float* f, int bf) {
  uint4 u;
  u.x = bf ? pack_bf16(f[0], f[1]) : pack_f16(f[0], f[1]);
  u.y = bf ? pack_bf16(f[2], f[3]) : pack_f16(f[2], f[3]);
  u.z = bf ? pack_bf16(f[4], f[5]) : pack_f16(f[4], f[5]);
  u.w = bf ? pack_bf16(f[6], f[7]) : pack_f16(f[6], f[7]);
  return u;
}

// NVSwitch multicast ("multimem") accesses: one load returns the sum of the addressed vector
// over all ranks' buffers (added inside the switch, fp32 accumulation for 16-bit types), one
// store writes every rank's copy.  The multicast address is a second mapping of the same
// memory, so accesses through it are ordered against ordinary ones with fence.proxy.alias.
__device__ __forceinline__ void fence_alias() { asm volatile("fence.proxy.alias;" ::: "memory"); }
__device__ __forceinline__ uint4 mm_ld_reduce_bf16(const void* p) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}
__device__ __forceinline__ uint4 mm_ld_reduce_f16(const void* p) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}
__device__ __forceinline__ float4 mm_ld_reduce_f32(const void* p) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(p) : "memory");
  return r;
}
__device__ __forceinline__ void mm_st(void* p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// One kernel = start barrier, reduce-scatter of this rank's slice (+ optimizer),
// all-gather by remote stores, end barrier.
__global__ void __launch_bounds__(512)
fused_step_kernel(const StepArgs a) {
  __shared__ int sm_flag;
  const int rank = a.emulate ? (int)blockIdx.y : a.rank;
  const int W = a.world;
  const int cta = blockIdx.x, G = gridDim.x;
  if (threadIdx.x == 0) sm_flag = 0;
  __syncthreads();
  const unsigned int epoch = dyn_value(a.epoch, a.epoch_base);
  if (W > 1 && !cta_barrier(a.pt, rank, W, 0, cta, epoch, a.status, &sm_flag)) return;
  float lr = a.lr, wd = a.wd, b1 = a.b1, b2 = a.b2, eps = a.eps, bc1 = a.bc1, bc2 = a.bc2, gscale = a.gscale;
  if (a.hyper_dev) {
    lr = __ldg(a.hyper_dev); wd = __ldg(a.hyper_dev + 1); b1 = __ldg(a.hyper_dev + 2); b2 = __ldg(a.hyper_dev + 3);
    eps = __ldg(a.hyper_dev + 4); bc1 = __ldg(a.hyper_dev + 5); bc2 = __ldg(a.hyper_dev + 6);
    gscale = __ldg(a.hyper_dev + 7);
  }
  if (a.mode == 1 && a.phase == 1) gscale = 1.f;   // the clip factor is applied in phase 2

  const int epv = a.dtype_bf16 == 2 ? 4 : 8;  // elements per 16-byte vector
  const long long L = a.n / W;          // elements in one rank's slice
  const long long nvec = L / epv;       // 16-byte vectors in the slice
  // interleave = 1: CTAs interleave at the granularity of one CTA-wide vector row (8 KB), so
  // that at any moment the whole grid works on one compact window of each array (keeps DRAM
  // pages open: 4.9 instead of 3.6 TB/s on one GPU).  interleave = 0: every CTA owns one
  // contiguous range.
  long long v0, v1, vstep;
  if (a.interleave) {
    v0 = (long long)cta * blockDim.x;
    v1 = nvec;
    vstep = (long long)G * blockDim.x;
  } else {
    const long long per = (nvec + G - 1) / G;
    v0 = (long long)cta * per;
    v1 = min(v0 + per, nvec);
    vstep = blockDim.x;
  }
  const long long slice_vec0 = (long long)rank * nvec;  // vector index of the slice start
  const float inv = gscale / (float)W;
  const int sidx = a.emulate ? rank : 0;
  float* master = a.master[sidx];
  float* mm = a.m[sidx];
  float* vv = a.v[sidx];

  const bool use_mc = a.mc != nullptr && W > 1 && !a.emulate;
  if (use_mc) fence_alias();
  if (a.dtype_bf16 == 2) {
    // fp32 all-reduce (mode 0): the same two-shot scheme on vectors of four floats
    for (long long i = v0 + threadIdx.x; i < v1; i += vstep) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (use_mc) {
        acc = mm_ld_reduce_f32((const float4*)((const char*)a.mc + a.grad_off) + slice_vec0 + i);
      } else {
        for (int p = 0; p < W; p++) {
          const float4 u = __ldcg((const float4*)((const char*)a.pt.base[p] + a.grad_off) + slice_vec0 + i);
          acc.x += u.x; acc.y += u.y; acc.z += u.z; acc.w += u.w;
        }
      }
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
      if (use_mc) {
        mm_st((float4*)((char*)a.mc + a.grad_off) + slice_vec0 + i,
              make_uint4(__float_as_uint(acc.x), __float_as_uint(acc.y), __float_as_uint(acc.z), __float_as_uint(acc.w)));
      } else {
        for (int p = 0; p < W; p++) {
          const int q = (rank + 1 + p) % W;
          ((float4*)((char*)a.pt.base[q] + a.grad_off))[slice_vec0 + i] = acc;
        }
      }
    }
    if (use_mc) fence_alias();
    if (W > 1) cta_barrier(a.pt, rank, W, 1, cta, epoch + 1, a.status, &sm_flag);
    return;
  }
  float sq_local = 0.f;
  const unsigned char* wmask = a.wd_mask[sidx];
  float* gsh = a.gshard[sidx];
  for (long long i = v0 + threadIdx.x; i < v1; i += vstep) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.f;
    if (a.mode == 1 && a.phase == 2) {
      // the averaged gradients were left in fp32 by phase 1; gscale (the clip factor) is known now
      const float4 g0 = *(const float4*)(gsh + i * 8), g1 = *(const float4*)(gsh + i * 8 + 4);
      acc[0] = g0.x * gscale; acc[1] = g0.y * gscale; acc[2] = g0.z * gscale; acc[3] = g0.w * gscale;
      acc[4] = g1.x * gscale; acc[5] = g1.y * gscale; acc[6] = g1.z * gscale; acc[7] = g1.w * gscale;
    } else {
      if (use_mc) {
        // the switch adds the W copies (fp32 accumulation) and returns the 16-bit sum
        const void* src = (const uint4*)((const char*)a.mc + a.grad_off) + slice_vec0 + i;
        const uint4 u = a.dtype_bf16 ? mm_ld_reduce_bf16(src) : mm_ld_reduce_f16(src);
        unpack8(u, acc, a.dtype_bf16);
      } else {
        // fixed rank order => the sum does not depend on who computes it or when
        for (int p = 0; p < W; p++) {
          const uint4* src = (const uint4*)((const char*)a.pt.base[p] + a.grad_off) + slice_vec0 + i;
          uint4 u = __ldcg(src);  // L2 only: a peer's data is never served from this SM's L1
          float f[8];
          unpack8(u, f, a.dtype_bf16);
#pragma unroll
          for (int j = 0; j < 8; j++) acc[j] += f[j];
        }
      }
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] *= inv;
    }
    if (a.mode == 1 && a.phase == 1) {
      *(float4*)(gsh + i * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *(float4*)(gsh + i * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
      for (int j = 0; j < 8; j++) sq_local += acc[j] * acc[j];
      continue;
    }
    uint4 out;
    long long dst_off;
    if (a.mode == 0) {
      out = pack8(acc, a.dtype_bf16);
      dst_off = a.grad_off;
    } else {
      float4* mp = (float4*)(master + i * 8);
      float4* m4 = (float4*)(mm + i * 8);
      float pw[8], pm[8], pv[8];
      *(float4*)&pw[0] = mp[0]; *(float4*)&pw[4] = mp[1];
      *(float4*)&pm[0] = m4[0]; *(float4*)&pm[4] = m4[1];
      const float wdv = (wmask == nullptr || wmask[i]) ? wd : 0.f;
      if (a.opt_kind == 0) {
        float4* v4 = (float4*)(vv + i * 8);
        *(float4*)&pv[0] = v4[0]; *(float4*)&pv[4] = v4[1];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float g = acc[j];
          float p = pw[j];
          p -= lr * wdv * p;  // decoupled decay first, like optim/adamw.go:77-81
          float m_ = b1 * pm[j] + (1.f - b1) * g;
          float v_ = b2 * pv[j] + (1.f - b2) * g * g;
          p -= lr * (m_ / bc1) / (sqrtf(v_ / bc2) + eps);
          pw[j] = p; pm[j] = m_; pv[j] = v_;
        }
        v4[0] = *(float4*)&pv[0]; v4[1] = *(float4*)&pv[4];
      } else if (a.opt_kind == 1) {
        // SGD with momentum b1 and coupled weight decay (optim/sgd.go:38-58): g += wd p; v = mu v + g; p -= lr v
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const float g = acc[j] + wdv * pw[j];
          const float v_ = b1 * pm[j] + g;
          pw[j] -= lr * v_;
          pm[j] = v_;
        }
      } else {
        // Lion (optim/lion.go:61-76): c = b1 m + (1-b1) g; p -= lr (sign(c) + wd p); m = b2 m + (1-b2) g
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const float g = acc[j];
          const float c = b1 * pm[j] + (1.f - b1) * g;
          const float sg = c > 0.f ? 1.f : (c < 0.f ? -1.f : 0.f);
          pw[j] -= lr * (sg + wdv * pw[j]);
          pm[j] = b2 * pm[j] + (1.f - b2) * g;
        }
      }
      mp[0] = *(float4*)&pw[0]; mp[1] = *(float4*)&pw[4];
      m4[0] = *(float4*)&pm[0]; m4[1] = *(float4*)&pm[4];
      out = pack8(pw, a.dtype_bf16);
      dst_off = a.param_off;
    }
    if (use_mc) {
      mm_st((uint4*)((char*)a.mc + dst_off) + slice_vec0 + i, out);   // every rank's copy in one store
    } else {
      for (int p = 0; p < W; p++) {
        // own copy last-to-first makes no difference; start with the next rank to spread traffic
        const int q = (rank + 1 + p) % W;
        uint4* dst = (uint4*)((char*)a.pt.base[q] + dst_off) + slice_vec0 + i;
        *dst = out;
      }
    }
  }
  if (a.mode == 1 && a.phase == 1) {
    // per-CTA sum of squares in a fixed order (block_sum is a fixed tree): reproducible
    __shared__ float red[32];
    const float tot = block_sum(sq_local, red);
    if (threadIdx.x == 0) a.sqpart[sidx][cta] = tot;
  }
  if (use_mc) fence_alias();
  if (W > 1) cta_barrier(a.pt, rank, W, 1, cta, epoch + 1, a.status, &sm_flag);
}

// One-shot all-reduce for short vectors: every rank pushes its vector into slot [parity][rank]
// of every peer, ONE barrier, then every rank adds the W slots in rank order and writes the
// result over its own vector.  The two slot sets alternate from call to call, so no second
// barrier is needed before the slots are reused: a rank can only reach call n+2 (which reuses
// the set of call n) after every peer has signalled in call n+1, i.e. has finished call n.
struct OneShotArgs {
  PeerTable pt;
  int rank, world, emulate;
  long long data_off;   // byte offset of the vector inside the symmetric buffer (in place)
  long long slot_off;   // byte offset of the slot area: 2 sets x world slots x slot_bytes
  long long slot_bytes; // bytes per slot (>= n * element size, multiple of 16)
  long long nvec;       // 16-byte vectors in the vector
  int dtype;            // 0 fp16, 1 bf16, 2 fp32
  float scale;          // applied to the sum (1/W for the mean)
  unsigned int epoch;
  const unsigned int* epoch_base;
  int* status;
};

__global__ void __launch_bounds__(256)
oneshot_allreduce_kernel(const OneShotArgs a) {
  __shared__ int sm_flag;
  const int rank = a.emulate ? (int)blockIdx.y : a.rank;
  const int W = a.world;
  const int cta = blockIdx.x, G = gridDim.x;
  if (threadIdx.x == 0) sm_flag = 0;
  __syncthreads();
  const unsigned int epoch = dyn_value(a.epoch, a.epoch_base);
  const long long set_off = a.slot_off + (long long)(epoch & 1u) * W * a.slot_bytes;
  const uint4* mine = (const uint4*)((const char*)a.pt.base[rank] + a.data_off);
  const long long per = (a.nvec + G - 1) / G;
  const long long v0 = (long long)cta * per, v1 = min(v0 + per, a.nvec);
  for (long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    const uint4 u = mine[i];
    for (int p = 0; p < W; p++) {
      const int q = (rank + 1 + p) % W;
      ((uint4*)((char*)a.pt.base[q] + set_off + (long long)rank * a.slot_bytes))[i] = u;
    }
  }
  if (!cta_barrier(a.pt, rank, W, 9, cta, epoch, a.status, &sm_flag)) return;
  const char* slots = (const char*)a.pt.base[rank] + set_off;
  uint4* outp = (uint4*)((char*)a.pt.base[rank] + a.data_off);
  for (long long i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    if (a.dtype == 2) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < W; p++) {
        const float4 u = __ldcg((const float4*)(slots + (long long)p * a.slot_bytes) + i);
        acc.x += u.x; acc.y += u.y; acc.z += u.z; acc.w += u.w;
      }
      acc.x *= a.scale; acc.y *= a.scale; acc.z *= a.scale; acc.w *= a.scale;
      ((float4*)outp)[i] = acc;
    } else {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] = 0.f;
      for (int p = 0; p < W; p++) {
        const uint4 u = __ldcg((const uint4*)(slots + (long long)p * a.slot_bytes) + i);
        float f[8];
        unpack8(u, f, a.dtype);
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] += f[j];
      }
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] *= a.scale;
      outp[i] = pack8(acc, a.dtype);
    }
  }
}

struct SmallArgs {
  PeerTable pt;
  int rank, world, emulate;
  long long slot_off;  // byte offset of the exchange area: world slots of n floats
  int n;
  unsigned int epoch;
  const unsigned int* epoch_base;
  float* io[kMaxWorld];  // in/out vector per emulated rank (index 0 in real runs)
  int* status;
};

// One-shot all-reduce-sum of a short fp32 vector: every rank stores its vector
// into slot[rank] of every peer, then sums the slots in rank order.
__global__ void __launch_bounds__(256)
allreduce_small_kernel(const SmallArgs a) {
  __shared__ int sm_flag;
  const int rank = a.emulate ? (int)blockIdx.y : a.rank;
  const int W = a.world;
  if (threadIdx.x == 0) sm_flag = 0;
  __syncthreads();
  float* io = a.io[a.emulate ? rank : 0];
  for (int p = 0; p < W; p++) {
    float* slot = (float*)((char*)a.pt.base[p] + a.slot_off) + (long long)rank * a.n;
    for (int i = threadIdx.x; i < a.n; i += blockDim.x) slot[i] = io[i];
  }
  const unsigned int epoch = dyn_value(a.epoch, a.epoch_base);
  if (!cta_barrier(a.pt, rank, W, 2, 0, epoch, a.status, &sm_flag)) return;
  const float* mine = (const float*)((const char*)a.pt.base[rank] + a.slot_off);
  for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
    float s = 0.f;
    for (int p = 0; p < W; p++) s += __ldcg(mine + (long long)p * a.n + i);
    io[i] = s;
  }
  // slots may be reused by the next call only after everyone has read them
  cta_barrier(a.pt, rank, W, 3, 0, epoch + 1, a.status, &sm_flag);
}

struct BcastArgs {
  PeerTable pt;
  int rank, world, emulate, root;
  long long off, bytes;
  unsigned int epoch;
  const unsigned int* epoch_base;
  int* status;
};

// Root pushes [off, off+bytes) of its symmetric buffer into every peer's.
__global__ void __launch_bounds__(512)
broadcast_kernel(const BcastArgs a) {
  __shared__ int sm_flag;
  const int rank = a.emulate ? (int)blockIdx.y : a.rank;
  const int W = a.world;
  const int cta = blockIdx.x, G = gridDim.x;
  if (threadIdx.x == 0) sm_flag = 0;
  __syncthreads();
  // everyone must have finished with the old contents before root overwrites them
  const unsigned int epoch = dyn_value(a.epoch, a.epoch_base);
  if (!cta_barrier(a.pt, rank, W, 4, cta, epoch, a.status, &sm_flag)) return;
  if (rank == a.root) {
    const long long nvec = a.bytes / 16;
    const uint4* src = (const uint4*)((const char*)a.pt.base[rank] + a.off);
    for (long long i = (long long)cta * blockDim.x + threadIdx.x; i < nvec; i += (long long)G * blockDim.x) {
      uint4 u = src[i];
      for (int p = 0; p < W; p++)
        if (p != rank) ((uint4*)((char*)a.pt.base[p] + a.off))[i] = u;
    }
  }
  cta_barrier(a.pt, rank, W, 5, cta, epoch + 1, a.status, &sm_flag);
}

__global__ void barrier_kernel(const PeerTable pt, int rank_arg, int world, int emulate,
                               unsigned int epoch, const unsigned int* epoch_base, int* status) {
  __shared__ int sm_flag;
  const int rank = emulate ? (int)blockIdx.y : rank_arg;
  if (threadIdx.x == 0) sm_flag = 0;
  __syncthreads();
  cta_barrier(pt, rank, world, 6, 0, dyn_value(epoch, epoch_base), status, &sm_flag);
}

// Wait for a flag that nobody sets: used by tests of the time-out path.  budget_ns
// bounds the wait; the kernel then records ST_COMM_TIMEOUT and returns.
__global__ void wait_flag_kernel(const unsigned int* flag, unsigned int want, unsigned long long budget_ns,
                                 int* status) {
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(flag) != want) {
    if (globaltimer_ns() - t0 > budget_ns) {
      set_status(status, ST_COMM_TIMEOUT, 999);
      return;
    }
  }
}

int launch_maybe_coop(const void* kern, dim3 grid, dim3 block, void** args, int emulate, cudaStream_t s) {
  if (emulate) {
    // emulated ranks wait on each other inside one launch: all CTAs must be co-resident
    GB_CUDA_OK(cudaLaunchCooperativeKernel(kern, grid, block, args, 0, s));
  } else {
    GB_CUDA_OK(cudaLaunchKernel(kern, grid, block, args, 0, s));
  }
  return gbh::E_OK;
}

}  // namespace

GB_EXPORT long long gb_comm_flag_bytes() { return (long long)kFlagBytes; }
GB_EXPORT int gb_comm_max_world() { return kMaxWorld; }
GB_EXPORT int gb_comm_max_ctas() { return kMaxCtas; }

// Allocates this rank's symmetric buffer (flag area + data_bytes), zeroes the
// flags and writes the 64-byte IPC handle to handle_out.  Returns the base.
GB_EXPORT int gb_comm_alloc(long long data_bytes, void** base_out, void* handle_out) {
  if (g_comm.local != nullptr) {
    gbh::set_error("gb_comm_alloc: a symmetric buffer already exists; call gb_comm_free first");
    return gbh::E_BAD_ARG;
  }
  size_t bytes = kFlagBytes + (size_t)data_bytes;
  void* p = nullptr;
  GB_CUDA_OK(cudaMalloc(&p, bytes));
  GB_CUDA_OK(cudaMemset(p, 0, kFlagBytes));
  GB_CUDA_OK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  GB_CUDA_OK(cudaIpcGetMemHandle(&h, p));
  memcpy(handle_out, &h, sizeof(h));
  g_comm.local = p;
  g_comm.bytes = bytes;
  g_comm.epoch = 0;
  *base_out = p;
  return gbh::E_OK;
}

// Maps every peer's buffer.  handles: world x 64 bytes, in rank order.
GB_EXPORT int gb_comm_open(int rank, int world, const void* handles) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) {
    gbh::set_error("gb_comm_open: bad rank/world %d/%d", rank, world);
    return gbh::E_BAD_ARG;
  }
  g_comm.rank = rank;
  g_comm.world = world;
  for (int p = 0; p < world; p++) {
    if (p == rank) {
      g_comm.peers.base[p] = g_comm.local;
      continue;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char*)handles + 64 * p, sizeof(h));
    void* q = nullptr;
    GB_CUDA_OK(cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess));
    g_comm.peers.base[p] = q;
    g_comm.opened[p] = true;
  }
  return gbh::E_OK;
}

// Single-process set-up for tests: `world` emulated ranks whose buffers are the
// given device pointers (all on the current GPU).
GB_EXPORT int gb_comm_emulate(int world, void* const* bases) {
  if (world < 1 || world > kMaxWorld) {
    gbh::set_error("gb_comm_emulate: bad world %d", world);
    return gbh::E_BAD_ARG;
  }
  g_comm.rank = 0;
  g_comm.world = world;
  for (int p = 0; p < world; p++) g_comm.peers.base[p] = bases[p];
  g_comm.epoch = 0;
  return gbh::E_OK;
}

// Adopts symmetric buffers that the caller has already mapped (for example through a virtual-
// memory allocator that also provides an NVSwitch multicast mapping).  bases: every rank's buffer
// as mapped in this process, in rank order; mc_base: the multicast alias, or null.  The buffers
// start with gb_comm_flag_bytes() bytes of flags, which the caller has zeroed.
GB_EXPORT int gb_comm_attach(int rank, int world, void* const* bases, void* mc_base) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) {
    gbh::set_error("gb_comm_attach: bad rank/world %d/%d", rank, world);
    return gbh::E_BAD_ARG;
  }
  if (g_comm.local != nullptr) {
    gbh::set_error("gb_comm_attach: a symmetric buffer already exists; call gb_comm_free first");
    return gbh::E_BAD_ARG;
  }
  g_comm.rank = rank;
  g_comm.world = world;
  for (int p = 0; p < world; p++) g_comm.peers.base[p] = bases[p];
  g_comm.mc_base = mc_base;
  g_comm.attached = true;
  g_comm.epoch = 0;
  return gbh::E_OK;
}
GB_EXPORT int gb_comm_has_multicast() { return g_comm.mc_base != nullptr; }
// 1 (default): reductions and broadcasts of the fused step go through the multicast mapping when
// one is attached; 0: plain peer loads and stores in fixed rank order (bit-reproducible sums).
GB_EXPORT int gb_comm_multimem(int on) {
  g_use_multimem = on;
  return gbh::E_OK;
}

GB_EXPORT int gb_comm_free() {
  if (g_comm.attached) {
    for (int p = 0; p < kMaxWorld; p++) g_comm.peers.base[p] = nullptr;
    g_comm.mc_base = nullptr;
    g_comm.attached = false;
    g_comm.world = 1;
    g_comm.rank = 0;
    return gbh::E_OK;
  }
  for (int p = 0; p < kMaxWorld; p++) {
    if (g_comm.opened[p]) {
      cudaIpcCloseMemHandle(g_comm.peers.base[p]);
      g_comm.opened[p] = false;
    }
    g_comm.peers.base[p] = nullptr;
  }
  if (g_comm.local) cudaFree(g_comm.local);
  g_comm.local = nullptr;
  g_comm.world = 1;
  g_comm.rank = 0;
  return gbh::E_OK;
}

static unsigned int next_epochs(int count) {
  if (g_comm.cap_bases) {            // capturing: relative to a base the host supplies per replay
    const unsigned int e = g_comm.cap_epochs;
    g_comm.cap_epochs += count;
    return e;
  }
  unsigned int e = g_comm.epoch + 1;
  g_comm.epoch += count;
  return e;
}
static unsigned int next_serials(int count) {
  if (g_comm.cap_bases) {
    const unsigned int e = g_comm.cap_serials;
    g_comm.cap_serials += count;
    return e;
  }
  unsigned int e = g_comm.serial + 1;
  g_comm.serial += count;
  return e;
}

namespace gbh {
void comm_get(gbc::PeerTable* pt, int* rank, int* world) {
  *pt = g_comm.peers;
  *rank = g_comm.rank;
  *world = g_comm.world;
}
unsigned int comm_next_epochs(int count) { return next_epochs(count); }
unsigned int comm_next_serials(int count) { return next_serials(count); }
const unsigned int* comm_epoch_base_ptr() { return g_comm.cap_bases; }
const unsigned int* comm_serial_base_ptr() { return g_comm.cap_bases ? g_comm.cap_bases + 1 : nullptr; }
}  // namespace gbh

// Capture mode for CUDA graphs.  Between begin and end, every kernel that uses barrier epochs
// or local serial numbers is launched with values counted from zero plus a pointer to
// `bases` (two device words: epoch base, serial base) that it reads when it runs.  `end`
// reports how many of each the captured work consumes; before every replay the caller
// reserves that many with gb_comm_reserve and writes the returned bases into `bases`.
GB_EXPORT int gb_comm_capture_begin(unsigned int* bases) {
  if (g_comm.cap_bases) {
    gbh::set_error("gb_comm_capture_begin: a capture is already open");
    return gbh::E_BAD_ARG;
  }
  g_comm.cap_bases = bases;
  g_comm.cap_epochs = g_comm.cap_serials = 0;
  return gbh::E_OK;
}
GB_EXPORT int gb_comm_capture_end(unsigned int* counts_out) {
  counts_out[0] = g_comm.cap_epochs;
  counts_out[1] = g_comm.cap_serials;
  g_comm.cap_bases = nullptr;
  return gbh::E_OK;
}
// Reserves `epochs` barrier epochs and `serials` serial numbers; bases_out receives the first of each.
GB_EXPORT int gb_comm_reserve(unsigned int epochs, unsigned int serials, unsigned int* bases_out) {
  bases_out[0] = g_comm.epoch + 1;
  bases_out[1] = g_comm.serial + 1;
  g_comm.epoch += epochs;
  g_comm.serial += serials;
  return gbh::E_OK;
}

// Work mapping of the fused step: 1 interleaved rows, 0 contiguous ranges, -1 (default)
// interleaved on one GPU (4.9 vs 3.6 TB/s measured) and contiguous with peers (steady-state
// steps of the 12-layer LM on eight GPUs: 19.5 ms contiguous, 20.0 ms interleaved).
int g_interleave = -1;
GB_EXPORT int gb_comm_tune(int interleave) {
  g_interleave = interleave;
  return 0;
}

// Fused bucket step (see the top of the file).  Offsets are bytes from the
// start of the symmetric buffer (flag area included).  n: elements, a multiple
// of world*8.  mode 0: mean of the gradients written to every rank; mode 1:
// sharded AdamW (master/m/v: this rank's shard of the bucket, n/world floats
// each) and all-gather of the 16-bit parameters.  hyper: {lr, wd, b1, b2, eps,
// bc1, bc2, gscale}; hyper_dev: when not null, a device copy of the same eight
// floats that the kernel reads when it runs (a captured launch then follows the
// values the host writes before each replay).  emulate != 0: master/m/v are
// arrays of `world` pointers.
// opt: {kind (0 AdamW, 1 SGD with momentum = hyper[2], 2 Lion), phase (0 whole step, 1 reduce-scatter
// into gshard + per-CTA sums of squares into sqpart, 2 update from gshard + all-gather)}.  wd_mask: one
// byte per 8 shard elements (0 = no weight decay) or null; gshard: n/world floats; sqpart: `ctas` floats.
// The three pointer arguments are arrays of `world` pointers when emulating, like master / m / v.
GB_EXPORT int gb_comm_fused_step2(int mode, int dtype_bf16, long long grad_off, long long param_off,
                                  long long n, float* const* master, float* const* m, float* const* v,
                                  const float* hyper, const float* hyper_dev, int opt_kind, int phase,
                                  const unsigned char* const* wd_mask, float* const* gshard,
                                  float* const* sqpart, int ctas, int emulate, void* stream) {
  const int W = g_comm.world;
  if (n % ((long long)W * 8) != 0) {
    gbh::set_error("gb_comm_fused_step: bucket length %lld is not a multiple of world*8", n);
    return gbh::E_BAD_ARG;
  }
  if (dtype_bf16 == 2 && mode != 0) {
    gbh::set_error("gb_comm_fused_step: fp32 buckets support the all-reduce mode only");
    return gbh::E_BAD_ARG;
  }
  if (opt_kind < 0 || opt_kind > 2 || phase < 0 || phase > 2 || (phase != 0 && (mode != 1 || gshard == nullptr)) ||
      (phase == 1 && sqpart == nullptr)) {
    gbh::set_error("gb_comm_fused_step: bad optimizer kind / phase arguments");
    return gbh::E_BAD_ARG;
  }
  if (ctas < 1) ctas = 1;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (emulate && ctas * W > 128) ctas = 128 / W;
  StepArgs a;
  memset(&a, 0, sizeof(a));
  a.pt = g_comm.peers;
  a.rank = g_comm.rank; a.world = W; a.emulate = emulate;
  a.grad_off = grad_off; a.param_off = param_off; a.n = n; a.mode = mode; a.dtype_bf16 = dtype_bf16;
  a.interleave = g_interleave < 0 ? (W == 1) : (g_interleave != 0);
  a.epoch = W > 1 ? next_epochs(2) : 0;
  a.epoch_base = g_comm.cap_bases;
  a.hyper_dev = hyper_dev;
  a.opt_kind = opt_kind; a.phase = phase;
  // measured on eight GPUs: the multicast path wins from about 4 MiB (835 against 628 GB/s bus at
  // 1 GiB), plain peer accesses below (30 against 40 us at 1 MiB)
  a.mc = (g_use_multimem && n * (dtype_bf16 == 2 ? 4 : 2) >= (2LL << 20)) ? g_comm.mc_base : nullptr;
  const int ns = emulate ? W : 1;
  for (int i = 0; i < ns; i++) {
    a.master[i] = master ? master[i] : nullptr;
    a.m[i] = m ? m[i] : nullptr;
    a.v[i] = v ? v[i] : nullptr;
    a.wd_mask[i] = wd_mask ? wd_mask[i] : nullptr;
    a.gshard[i] = gshard ? gshard[i] : nullptr;
    a.sqpart[i] = sqpart ? sqpart[i] : nullptr;
  }
  a.lr = hyper[0]; a.wd = hyper[1]; a.b1 = hyper[2]; a.b2 = hyper[3]; a.eps = hyper[4];
  a.bc1 = hyper[5]; a.bc2 = hyper[6]; a.gscale = hyper[7];
  a.status = gbh::status_ptr();
  void* args[] = {&a};
  dim3 grid(ctas, emulate ? W : 1);
  return launch_maybe_coop((const void*)fused_step_kernel, grid, dim3(512), args, emulate && W > 1,
                           (cudaStream_t)stream);
}

GB_EXPORT int gb_comm_fused_step(int mode, int dtype_bf16, long long grad_off, long long param_off,
                                 long long n, float* const* master, float* const* m, float* const* v,
                                 const float* hyper, const float* hyper_dev, int ctas, int emulate,
                                 void* stream) {
  return gb_comm_fused_step2(mode, dtype_bf16, grad_off, param_off, n, master, m, v, hyper, hyper_dev, 0, 0, nullptr,
                             nullptr, nullptr, ctas, emulate, stream);
}

namespace {
// Gradient clipping by global norm (optim/clip.go:23-65): scale = max_norm / (norm + 1e-6), applied only when
// below 1.  sq: `count` partial sums of squares (already summed over ranks when there are several); writes the
// factor to hyper_dev[7] and the norm to norm_out.
__global__ void clip_scale_kernel(const float* __restrict__ sq, int count, float max_norm, float* hyper_dev,
                                  float* norm_out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) s += sq[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float norm = sqrtf(s);
    const float scale = max_norm / (norm + 1e-6f);
    hyper_dev[7] = scale < 1.f ? scale : 1.f;
    if (norm_out) *norm_out = norm;
  }
}
// out[0] = sum of `count` floats in index order (one thread: the order is part of the contract)
__global__ void sum_partials_kernel(const float* __restrict__ p, int count, float* out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) s += p[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s;
}
}  // namespace

// out[0] = sum of count floats (the per-CTA sums of squares of this rank's shards).
GB_EXPORT int gb_comm_sum_partials(const float* p, int count, float* out, void* stream) {
  if (p == nullptr || out == nullptr || count < 1) {
    gbh::set_error("gb_comm_sum_partials: null argument");
    return gbh::E_BAD_ARG;
  }
  sum_partials_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(p, count, out);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
// hyper_dev[7] = min(1, max_norm / (sqrt(sum sq[0..count)) + 1e-6)); norm_out (optional) = the norm.
GB_EXPORT int gb_comm_clip_scale(const float* sq, int count, float max_norm, float* hyper_dev, float* norm_out,
                                 void* stream) {
  if (sq == nullptr || hyper_dev == nullptr || count < 1) {
    gbh::set_error("gb_comm_clip_scale: null argument");
    return gbh::E_BAD_ARG;
  }
  clip_scale_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(sq, count, max_norm, hyper_dev, norm_out);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// One-shot all-reduce of a short vector, in place at data_off (see the kernel).  n elements of
// dtype (0 fp16, 1 bf16, 2 fp32), n * element size a multiple of 16; the slot area at slot_off
// must hold 2 * world * slot_bytes bytes with slot_bytes >= n * element size.
GB_EXPORT int gb_comm_allreduce_oneshot(int dtype, long long data_off, long long n, long long slot_off,
                                        long long slot_bytes, float scale, int ctas, int emulate, void* stream) {
  const int W = g_comm.world;
  const long long esz = dtype == 2 ? 4 : 2;
  if ((n * esz) % 16 != 0 || slot_bytes % 16 != 0 || slot_bytes < n * esz || data_off % 16 != 0 || slot_off % 16 != 0) {
    gbh::set_error("gb_comm_allreduce_oneshot: sizes and offsets must be multiples of 16 bytes and fit the slots");
    return gbh::E_BAD_ARG;
  }
  if (ctas < 1) ctas = 1;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (emulate && ctas * W > 128) ctas = 128 / W;
  OneShotArgs a;
  memset(&a, 0, sizeof(a));
  a.pt = g_comm.peers;
  a.rank = g_comm.rank; a.world = W; a.emulate = emulate;
  a.data_off = data_off; a.slot_off = slot_off; a.slot_bytes = slot_bytes; a.nvec = n * esz / 16;
  a.dtype = dtype; a.scale = scale;
  a.epoch = next_epochs(1);
  a.epoch_base = g_comm.cap_bases;
  a.status = gbh::status_ptr();
  void* args[] = {&a};
  return launch_maybe_coop((const void*)oneshot_allreduce_kernel, dim3(ctas, emulate ? W : 1), dim3(256), args,
                           emulate && W > 1, (cudaStream_t)stream);
}

// In-place sum over ranks of an fp32 vector of n <= 4096 elements.  slot_off:
// byte offset of an exchange area of world*n floats inside the symmetric buffer.
GB_EXPORT int gb_comm_allreduce_small(float* const* io, int n, long long slot_off, int emulate,
                                      void* stream) {
  const int W = g_comm.world;
  if (W == 1) return gbh::E_OK;
  SmallArgs a;
  memset(&a, 0, sizeof(a));
  a.pt = g_comm.peers;
  a.rank = g_comm.rank; a.world = W; a.emulate = emulate;
  a.slot_off = slot_off; a.n = n;
  a.epoch = next_epochs(2);
  a.epoch_base = g_comm.cap_bases;
  for (int i = 0; i < (emulate ? W : 1); i++) a.io[i] = io[i];
  a.status = gbh::status_ptr();
  void* args[] = {&a};
  return launch_maybe_coop((const void*)allreduce_small_kernel, dim3(1, emulate ? W : 1), dim3(256), args,
                           emulate, (cudaStream_t)stream);
}

GB_EXPORT int gb_comm_broadcast(int root, long long off, long long bytes, int ctas, int emulate,
                                void* stream) {
  const int W = g_comm.world;
  if (W == 1) return gbh::E_OK;
  if (bytes % 16 != 0 || off % 16 != 0) {
    gbh::set_error("gb_comm_broadcast: offset and size must be multiples of 16 bytes");
    return gbh::E_BAD_ARG;
  }
  if (ctas < 1) ctas = 1;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (emulate && ctas * W > 128) ctas = 128 / W;
  BcastArgs a;
  memset(&a, 0, sizeof(a));
  a.pt = g_comm.peers;
  a.rank = g_comm.rank; a.world = W; a.emulate = emulate; a.root = root;
  a.off = off; a.bytes = bytes;
  a.epoch = next_epochs(2);
  a.epoch_base = g_comm.cap_bases;
  a.status = gbh::status_ptr();
  void* args[] = {&a};
  return launch_maybe_coop((const void*)broadcast_kernel, dim3(ctas, emulate ? W : 1), dim3(512), args,
                           emulate, (cudaStream_t)stream);
}

GB_EXPORT int gb_comm_barrier(int emulate, void* stream) {
  const int W = g_comm.world;
  if (W == 1) return gbh::E_OK;
  PeerTable pt = g_comm.peers;
  int rank = g_comm.rank, world = W, emu = emulate;
  unsigned int epoch = next_epochs(1);
  const unsigned int* epoch_base = g_comm.cap_bases;
  int* status = gbh::status_ptr();
  void* args[] = {&pt, &rank, &world, &emu, &epoch, &epoch_base, &status};
  return launch_maybe_coop((const void*)barrier_kernel, dim3(1, emulate ? W : 1), dim3(32), args, emulate,
                           (cudaStream_t)stream);
}

// Launches a single thread that waits (at most budget_ns) for *flag == want.
// With a flag nobody sets this exercises the time-out path: the kernel returns
// normally and the status word holds ST_COMM_TIMEOUT.
GB_EXPORT int gb_comm_wait_flag(const unsigned int* flag, unsigned int want, long long budget_ns,
                                void* stream) {
  wait_flag_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, want, (unsigned long long)budget_ns,
                                                      gbh::status_ptr());
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
