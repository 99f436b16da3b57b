// Kernels that fuse data-parallel communication with the arithmetic around it, over NVLink / NVSwitch peer
// memory.  Every rank maps every peer's window (gradient buffers, parameter buffers, flag words) into its
// own address space; kernels then load from and store to peers directly (or through an NVSwitch multicast
// address with multimem instructions), so no NCCL call is on these paths.
//
//  * fbam_rs_adamw_ag     — gradient reduce-scatter + bf16→fp32 cast/scale + sharded AdamW + parameter
//                           all-gather, one launch per flat bucket: each rank sums ITS slice of the bucket
//                           over all peers' gradient buffers, updates its slice of the fp32 master / m / v,
//                           and writes the rounded parameters into every peer's parameter buffer.
//  * fbam_reduce_pull     — sum of all peers' gradients for a range (Muon: the owner of a matrix gathers its
//                           gradient), fused with the momentum update and the Frobenius-norm partial sum.
//  * fbam_push_shard      — copy a range of a local buffer into every peer's buffer and raise a per-source
//                           ready flag (all-gather whose consumers wait per shard, e.g. the flag-gated GEMM).
//  * fbam_reduce_slots    — owner-side half of GEMM -> reduce-scatter: waits for all peers' partial tiles (stored
//                           into per-source slots by the GEMM epilogue or by peer copies) and sums the slots.
//  * fbam_peer_barrier    — stand-alone cross-GPU barrier on the flag words.
//  * fbam_ipc_*           — peer windows over CUDA IPC handles, for groups whose member processes change.
//
// Synchronisation is by epoch-tagged flag words in peer memory: a rank publishes epoch e by storing e into
// its slot of every peer's flag array (st.release.sys after a system-scope fence) and waits until all slots
// of its own array hold >= e (ld.acquire.sys).  Every wait is bounded; when it runs out the kernel records
// COMM_ERR_PEER_TIMEOUT plus the rank it was waiting for in `status` and returns, leaving the context usable.
//
// The reference reduces gradients with NCCL all-reduce calls on packed buffers and steps the optimizer afterwards
// (reference: src/main.cpp:3572-3713, ccl/src/ccl_nccl.cpp:197-232); these kernels replace that sequence.
#include "elem16.cuh"
#include <cuda_runtime.h>
#include <string.h>
#include <stdint.h>

#define FBAM_MAX_RANKS 8

struct PeerPtrs {
  void* p[FBAM_MAX_RANKS];
};

namespace {

enum { COMM_ERR_PEER_TIMEOUT = 301 };

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Bounded wait until flags[slot*MAX + r] >= epoch for every r < world.  `spin_limit` polls per rank.
__device__ __forceinline__ bool wait_all(const unsigned* my_flags, int slot, int world, unsigned epoch,
                                         unsigned spin_limit, int* status) {
  for (int r = 0; r < world; ++r) {
    const unsigned* f = my_flags + slot * FBAM_MAX_RANKS + r;
    unsigned spins = 0;
    while ((int)(ld_acquire_sys(f) - epoch) < 0) {
      if (++spins > spin_limit) {
        atomicExch(status, COMM_ERR_PEER_TIMEOUT + 1000 * (r + 1));
        return false;
      }
      __nanosleep(100);
    }
  }
  return true;
}

// Entry barrier: CTA 0 tells every peer that this rank has arrived; every CTA then waits on the LOCAL flag array
// until all peers have arrived.  CTAs do not depend on one another, so the grid need not be co-resident.
__device__ bool signal_and_wait(const PeerPtrs& flags, int rank, int world, int slot, unsigned epoch,
                                unsigned spin_limit, int* status) {
  int ok = 1;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        st_release_sys(reinterpret_cast<unsigned*>(flags.p[r]) + slot * FBAM_MAX_RANKS + rank, epoch);
    }
    ok = wait_all(reinterpret_cast<const unsigned*>(flags.p[rank]), slot, world, epoch, spin_limit, status) ? 1 : 0;
  }
  return __syncthreads_and(ok) != 0;
}

// Exit barrier: every CTA makes its writes visible and counts itself in; only the LAST CTA of the grid
// publishes this rank's completion to the peers and waits for theirs.  All other CTAs leave at once, so no CTA
// ever waits for a CTA of its own grid that may not have been scheduled yet.
__device__ void finish_and_wait(const PeerPtrs& flags, int rank, int world, int slot, unsigned epoch,
                                unsigned spin_limit, int* status, unsigned* local_arrive) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(local_arrive, 1u);
    if (prev + 1 == gridDim.x) {
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        st_release_sys(reinterpret_cast<unsigned*>(flags.p[r]) + slot * FBAM_MAX_RANKS + rank, epoch);
      wait_all(reinterpret_cast<const unsigned*>(flags.p[rank]), slot, world, epoch, spin_limit, status);
    }
  }
}

__device__ __forceinline__ void unpack_elem8(const uint4& raw, float* f) {
  const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = e22ff(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack_elem8(const float* f) {
  uint4 raw;
  elem2_t* h = reinterpret_cast<elem2_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = ff2e2(f[2 * i], f[2 * i + 1]);
  return raw;
}

struct AdamArgs {
  float lr, b1, b2, eps, wd, inv_bc1, inv_bc2, grad_scale;
};

// -------------------------------------------------------------------------------------------------
// reduce-scatter + AdamW + all-gather.  The shard [lo, hi) (element indices, multiples of 8) is this rank's.
// ELEM16 = parameters/gradients are 16-bit (the element type) with an fp32 master copy; otherwise they are fp32 (no master).
// MULTIMEM = gradients are summed by the switch (multimem.ld_reduce) and parameters broadcast by it
// (multimem.st) through the multicast addresses mc_grad / mc_param.
// -------------------------------------------------------------------------------------------------
template <bool ELEM16, bool MULTIMEM>
__global__ void __launch_bounds__(256)
rs_adamw_ag_kernel(PeerPtrs grads, PeerPtrs params, PeerPtrs flags, void* mc_grad, void* mc_param, float* m, float* v,
                   float* master, long long lo, long long hi, AdamArgs a, int rank, int world, unsigned epoch,
                   int sync, unsigned spin_limit, int* status, unsigned* arrive) {
  // phase 0: every rank's gradients are complete (this kernel is stream-ordered after the local backward)
  if (sync && !signal_and_wait(flags, rank, world, 0, epoch, spin_limit, status)) return;

  constexpr int VEC = ELEM16 ? 8 : 4;  // elements per 16-byte packet
  const long long packets = (hi - lo) / VEC;
  for (long long pk = (long long)blockIdx.x * blockDim.x + threadIdx.x; pk < packets;
       pk += (long long)gridDim.x * blockDim.x) {
    const long long i = lo + pk * VEC;
    float g[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) g[j] = 0.0f;
    if constexpr (MULTIMEM) {
      if constexpr (ELEM16) {
        uint4 raw;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4." ELEM_PTX "x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                     : "l"(reinterpret_cast<const elem_t*>(mc_grad) + i)
                     : "memory");
        unpack_elem8(raw, g);
      } else {
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(g[0]), "=f"(g[1]), "=f"(g[2]), "=f"(g[3])
                     : "l"(reinterpret_cast<const float*>(mc_grad) + i)
                     : "memory");
      }
    } else {
      // All peers' packets are requested before any is used: one NVLink round trip in flight per peer instead of
      // one after the other.  Fixed summation order (rank 0, 1, ...) on every rank: results do not depend on
      // who owns the shard.
      uint4 raw[FBAM_MAX_RANKS];
#pragma unroll
      for (int r = 0; r < FBAM_MAX_RANKS; ++r)
        if (r < world)
          raw[r] = ELEM16 ? ld_cg_v4(reinterpret_cast<const elem_t*>(grads.p[r]) + i)
                        : ld_cg_v4(reinterpret_cast<const float*>(grads.p[r]) + i);
#pragma unroll
      for (int r = 0; r < FBAM_MAX_RANKS; ++r) {
        if (r < world) {
          if constexpr (ELEM16) {
            float t[8];
            unpack_elem8(raw[r], t);
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] += t[j];
          } else {
            g[0] += __uint_as_float(raw[r].x); g[1] += __uint_as_float(raw[r].y);
            g[2] += __uint_as_float(raw[r].z); g[3] += __uint_as_float(raw[r].w);
          }
        }
      }
    }
    float w[VEC];
    if constexpr (ELEM16) {
      const float4 w0 = *reinterpret_cast<const float4*>(master + i), w1 = *reinterpret_cast<const float4*>(master + i + 4);
      w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
    } else {
      const float4 w0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(params.p[rank]) + i);
      w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
    }
    float mv[VEC], vv[VEC];  // optimizer state moves in 16-byte accesses
#pragma unroll
    for (int j = 0; j < VEC; j += 4) {
      const float4 tm = *reinterpret_cast<const float4*>(m + i + j), tv = *reinterpret_cast<const float4*>(v + i + j);
      mv[j] = tm.x; mv[j + 1] = tm.y; mv[j + 2] = tm.z; mv[j + 3] = tm.w;
      vv[j] = tv.x; vv[j + 1] = tv.y; vv[j + 2] = tv.z; vv[j + 3] = tv.w;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float gj = g[j] * a.grad_scale;
      mv[j] = a.b1 * mv[j] + (1.0f - a.b1) * gj;
      vv[j] = a.b2 * vv[j] + (1.0f - a.b2) * gj * gj;
      w[j] = w[j] * (1.0f - a.lr * a.wd) - a.lr * (mv[j] * a.inv_bc1) / (sqrtf(vv[j] * a.inv_bc2) + a.eps);
    }
#pragma unroll
    for (int j = 0; j < VEC; j += 4) {
      *reinterpret_cast<float4*>(m + i + j) = make_float4(mv[j], mv[j + 1], mv[j + 2], mv[j + 3]);
      *reinterpret_cast<float4*>(v + i + j) = make_float4(vv[j], vv[j + 1], vv[j + 2], vv[j + 3]);
    }
    uint4 out;
    if constexpr (ELEM16) {
      *reinterpret_cast<float4*>(master + i) = make_float4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<float4*>(master + i + 4) = make_float4(w[4], w[5], w[6], w[7]);
      out = pack_elem8(w);
    } else {
      out = make_uint4(__float_as_uint(w[0]), __float_as_uint(w[1]), __float_as_uint(w[2]), __float_as_uint(w[3]));
    }
    // all-gather: the updated packet goes to every rank's parameter buffer
    if constexpr (MULTIMEM) {
      void* dst = ELEM16 ? static_cast<void*>(reinterpret_cast<elem_t*>(mc_param) + i)
                       : static_cast<void*>(reinterpret_cast<float*>(mc_param) + i);
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst),
                   "f"(__uint_as_float(out.x)), "f"(__uint_as_float(out.y)), "f"(__uint_as_float(out.z)),
                   "f"(__uint_as_float(out.w))
                   : "memory");
    } else {
#pragma unroll
      for (int r = 0; r < FBAM_MAX_RANKS; ++r) {
        if (r < world) {
          void* dst = ELEM16 ? static_cast<void*>(reinterpret_cast<elem_t*>(params.p[r]) + i)
                           : static_cast<void*>(reinterpret_cast<float*>(params.p[r]) + i);
          *reinterpret_cast<uint4*>(dst) = out;
        }
      }
    }
  }
  // phase 1: every rank has written its shard everywhere (and has finished reading everyone's gradients)
  if (sync) finish_and_wait(flags, rank, world, 1, epoch, spin_limit, status, arrive);
}

// -------------------------------------------------------------------------------------------------
// Sum of all peers' gradients over [lo, hi) -> momentum buffer update -> bf16 update direction + Σ x².
// buf = mu*buf + (1 - mu)*g;  u = nesterov ? (1 - mu)*g + mu*buf : buf;  out_elem = u;  sumsq += Σ u²
// (the momentum buffer is an exponential moving average, as in the reference: src/optimizers.cpp:1204-1226)
// -------------------------------------------------------------------------------------------------
template <bool ELEM16>
__global__ void __launch_bounds__(256)
reduce_pull_kernel(PeerPtrs grads, float* momentum_buf, elem_t* out, float* sumsq, long long lo, long long hi, float mu,
                   int nesterov, float grad_scale, int world) {
  constexpr int VEC = ELEM16 ? 8 : 4;
  const long long packets = (hi - lo) / VEC;
  float local = 0.0f;
  for (long long pk = (long long)blockIdx.x * blockDim.x + threadIdx.x; pk < packets;
       pk += (long long)gridDim.x * blockDim.x) {
    const long long i = lo + pk * VEC;
    float g[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) g[j] = 0.0f;
    uint4 raw[FBAM_MAX_RANKS];  // every peer's packet is in flight before the first is used
#pragma unroll
    for (int r = 0; r < FBAM_MAX_RANKS; ++r)
      if (r < world)
        raw[r] = ELEM16 ? ld_cg_v4(reinterpret_cast<const elem_t*>(grads.p[r]) + i)
                      : ld_cg_v4(reinterpret_cast<const float*>(grads.p[r]) + i);
#pragma unroll
    for (int r = 0; r < FBAM_MAX_RANKS; ++r) {
      if (r < world) {
        if constexpr (ELEM16) {
          float t[8];
          unpack_elem8(raw[r], t);
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] += t[j];
        } else {
          g[0] += __uint_as_float(raw[r].x); g[1] += __uint_as_float(raw[r].y);
          g[2] += __uint_as_float(raw[r].z); g[3] += __uint_as_float(raw[r].w);
        }
      }
    }
    // momentum buffer and output are indexed from lo; lo is a multiple of VEC and both are 16-byte aligned
    float bufv[VEC], u[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j += 4) {
      const float4 t = *reinterpret_cast<const float4*>(momentum_buf + (i - lo) + j);
      bufv[j] = t.x; bufv[j + 1] = t.y; bufv[j + 2] = t.z; bufv[j + 3] = t.w;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float gj = g[j] * grad_scale * (1.0f - mu);
      bufv[j] = mu * bufv[j] + gj;
      u[j] = nesterov ? gj + mu * bufv[j] : bufv[j];
      local += u[j] * u[j];
    }
#pragma unroll
    for (int j = 0; j < VEC; j += 4)
      *reinterpret_cast<float4*>(momentum_buf + (i - lo) + j) = make_float4(bufv[j], bufv[j + 1], bufv[j + 2], bufv[j + 3]);
    if constexpr (ELEM16) {
      *reinterpret_cast<uint4*>(out + (i - lo)) = pack_elem8(u);
    } else {
      __align__(8) elem2_t h[2] = {ff2e2(u[0], u[1]), ff2e2(u[2], u[3])};
      *reinterpret_cast<uint2*>(out + (i - lo)) = *reinterpret_cast<uint2*>(h);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(sumsq, local);
}

// Copy [lo_bytes, hi_bytes) of the local buffer into every peer's buffer, then raise flag `slot`/rank.
__global__ void __launch_bounds__(256)
push_shard_kernel(PeerPtrs bufs, PeerPtrs flags, long long lo_bytes, long long hi_bytes, int rank, int world, int slot,
                  unsigned epoch, unsigned* arrive) {
  const long long packets = (hi_bytes - lo_bytes) / 16;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(bufs.p[rank]) + lo_bytes);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long pk = (long long)blockIdx.x * blockDim.x + threadIdx.x; pk < packets; pk += 4 * stride) {
    uint4 val[4];  // four independent loads in flight per thread
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (pk + u * stride < packets) val[u] = src[pk + u * stride];
#pragma unroll
    for (int r = 0; r < FBAM_MAX_RANKS; ++r) {
      if (r < world && r != rank) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(bufs.p[r]) + lo_bytes);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (pk + u * stride < packets) dst[pk + u * stride] = val[u];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(arrive, 1u);
    if (prev + 1 == gridDim.x) {  // last CTA: all of this grid's stores are ordered before the flag
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        st_release_sys(reinterpret_cast<unsigned*>(flags.p[r]) + slot * FBAM_MAX_RANKS + rank, epoch);
    }
  }
}

__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, int slot, unsigned epoch, unsigned spin_limit,
                                    int* status) {
  signal_and_wait(flags, rank, world, slot, epoch, spin_limit, status);
}

// Wait (bounded) until the local flags of `slot` reach `epoch`; sets status on timeout.
__global__ void wait_flags_kernel(const unsigned* my_flags, int slot, int world, unsigned epoch, unsigned spin_limit,
                                  int* status) {
  if (threadIdx.x == 0) wait_all(my_flags, slot, world, epoch, spin_limit, status);
}


// Owner-side half of the slot-form GEMM -> reduce-scatter: after every peer has announced that its partial tiles
// are stored (entry barrier on the flag words), sum the `world` bf16 slots of the local buffer in fp32.
__global__ void __launch_bounds__(256)
reduce_slots_kernel(const uint4* __restrict__ slots, uint4* __restrict__ out, long long packets_per_slot, int world,
                    PeerPtrs flags, int rank, int slot, unsigned epoch, unsigned spin_limit, int sync, int* status) {
  if (sync && !signal_and_wait(flags, rank, world, slot, epoch, spin_limit, status)) return;
  for (long long pk = (long long)blockIdx.x * blockDim.x + threadIdx.x; pk < packets_per_slot;
       pk += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      const uint4 raw = __ldcg(slots + (long long)r * packets_per_slot + pk);
      const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = e22ff(h[q]);
        acc[2 * q] += f.x;
        acc[2 * q + 1] += f.y;
      }
    }
    __align__(16) elem2_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) o[q] = ff2e2(acc[2 * q], acc[2 * q + 1]);
    out[pk] = *reinterpret_cast<uint4*>(o);
  }
}

int num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

}  // namespace

#define STREAM(s) reinterpret_cast<cudaStream_t>(s)

extern "C" {

int fbam_comm_max_ranks() { return FBAM_MAX_RANKS; }

// grads/params/flags: arrays of `world` device pointers (peer-mapped).  mc_grad/mc_param: multicast addresses
// or null (then plain peer loads/stores are used).  arrive: one zeroed unsigned in local memory.
// sync = 0 skips the cross-rank barriers (single-process emulation of several ranks, one launch per rank).
int fbam_rs_adamw_ag(void* const* grads, void* const* params, void* const* flags, void* mc_grad, void* mc_param,
                     float* m, float* v, float* master, long long lo, long long hi, int is_elem, float lr, float b1,
                     float b2, float eps, float wd, float bc1, float bc2, float grad_scale, int rank, int world,
                     unsigned epoch, int sync, unsigned spin_limit, int* status, unsigned* arrive, int max_ctas,
                     void* stream) {
  if (world < 1 || world > FBAM_MAX_RANKS || rank < 0 || rank >= world) return 1;
  const int vec = is_elem ? 8 : 4;
  if (lo % vec != 0 || hi % vec != 0 || hi < lo) return 1;
  if (is_elem && master == nullptr) return 1;
  if ((reinterpret_cast<uintptr_t>(m) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(master) & 15))
    return 1;
  PeerPtrs G{}, P{}, F{};
  for (int r = 0; r < world; ++r) {
    G.p[r] = grads[r];
    P.p[r] = params[r];
    F.p[r] = flags ? flags[r] : nullptr;
  }
  if (sync && flags == nullptr) return 1;
  AdamArgs a{lr, b1, b2, eps, wd, 1.0f / bc1, 1.0f / bc2, grad_scale};
  const long long packets = (hi - lo) / vec;
  int grid = (int)((packets + 255) / 256);
  int cap = max_ctas > 0 ? max_ctas : num_sms() * 4;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  cudaStream_t s = STREAM(stream);
  if (cudaMemsetAsync(arrive, 0, sizeof(unsigned), s) != cudaSuccess) return 5;
  const bool mm = mc_grad != nullptr && mc_param != nullptr;
#define LAUNCH(BF, MM)                                                                                              \
  rs_adamw_ag_kernel<BF, MM><<<grid, 256, 0, s>>>(G, P, F, mc_grad, mc_param, m, v, master, lo, hi, a, rank, world, \
                                                  epoch, sync, spin_limit, status, arrive)
  if (is_elem) { if (mm) LAUNCH(true, true); else LAUNCH(true, false); }
  else { if (mm) LAUNCH(false, true); else LAUNCH(false, false); }
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

int fbam_reduce_pull(void* const* grads, float* momentum_buf, void* out_elem, float* sumsq, long long lo, long long hi,
                     int is_elem, float mu, int nesterov, float grad_scale, int world, void* stream) {
  if (world < 1 || world > FBAM_MAX_RANKS) return 1;
  const int vec = is_elem ? 8 : 4;
  if (lo % vec != 0 || hi % vec != 0 || hi < lo) return 1;
  if ((reinterpret_cast<uintptr_t>(momentum_buf) & 15) || (reinterpret_cast<uintptr_t>(out_elem) & 15)) return 1;
  PeerPtrs G{};
  for (int r = 0; r < world; ++r) G.p[r] = grads[r];
  const long long packets = (hi - lo) / vec;
  int grid = (int)((packets + 255) / 256);
  if (grid > num_sms() * 4) grid = num_sms() * 4;
  if (grid < 1) grid = 1;
  if (is_elem)
    reduce_pull_kernel<true><<<grid, 256, 0, STREAM(stream)>>>(G, momentum_buf, (elem_t*)out_elem, sumsq, lo, hi, mu,
                                                               nesterov, grad_scale, world);
  else
    reduce_pull_kernel<false><<<grid, 256, 0, STREAM(stream)>>>(G, momentum_buf, (elem_t*)out_elem, sumsq, lo, hi, mu,
                                                                nesterov, grad_scale, world);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

int fbam_push_shard(void* const* bufs, void* const* flags, long long lo_bytes, long long hi_bytes, int rank, int world,
                    int slot, unsigned epoch, unsigned* arrive, void* stream) {
  if (world < 1 || world > FBAM_MAX_RANKS || lo_bytes % 16 != 0 || hi_bytes % 16 != 0) return 1;
  PeerPtrs B{}, F{};
  for (int r = 0; r < world; ++r) {
    B.p[r] = bufs[r];
    F.p[r] = flags[r];
  }
  const long long packets = (hi_bytes - lo_bytes) / 16;
  int grid = (int)((packets + 1023) / 1024);
  if (grid > num_sms() * 2) grid = num_sms() * 2;
  if (grid < 1) grid = 1;
  cudaStream_t s = STREAM(stream);
  if (cudaMemsetAsync(arrive, 0, sizeof(unsigned), s) != cudaSuccess) return 5;
  push_shard_kernel<<<grid, 256, 0, s>>>(B, F, lo_bytes, hi_bytes, rank, world, slot, epoch, arrive);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

int fbam_peer_barrier(void* const* flags, int rank, int world, int slot, unsigned epoch, unsigned spin_limit,
                      int* status, void* stream) {
  if (world < 1 || world > FBAM_MAX_RANKS) return 1;
  PeerPtrs F{};
  for (int r = 0; r < world; ++r) F.p[r] = flags[r];
  peer_barrier_kernel<<<1, 32, 0, STREAM(stream)>>>(F, rank, world, slot, epoch, spin_limit, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

int fbam_wait_flags(const void* my_flags, int slot, int world, unsigned epoch, unsigned spin_limit, int* status,
                    void* stream) {
  wait_flags_kernel<<<1, 32, 0, STREAM(stream)>>>((const unsigned*)my_flags, slot, world, epoch, spin_limit, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

// slots: local buffer [world][n_per_slot] bf16; out: n_per_slot bf16.  flags == null skips the entry barrier
// (single-process emulation).
int fbam_reduce_slots(const void* slots, void* out, long long n_per_slot, int world, void* const* flags, int rank,
                      int slot, unsigned epoch, unsigned spin_limit, int* status, void* stream) {
  if (world < 1 || world > FBAM_MAX_RANKS || n_per_slot % 8 != 0 || n_per_slot < 0) return 1;
  if ((reinterpret_cast<uintptr_t>(slots) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return 1;
  PeerPtrs F{};
  if (flags != nullptr)
    for (int r = 0; r < world; ++r) F.p[r] = flags[r];
  const long long packets = n_per_slot / 8;
  int grid = (int)((packets + 255) / 256);
  if (grid > num_sms() * 4) grid = num_sms() * 4;
  if (grid < 1) grid = 1;
  reduce_slots_kernel<<<grid, 256, 0, STREAM(stream)>>>((const uint4*)slots, (uint4*)out, packets, world, F, rank, slot,
                                                        epoch, spin_limit, flags != nullptr, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

// Device-to-device copy on `stream` by the copy engines (cudaMemcpyAsync); either side may be a peer mapping.
int fbam_copy_async(void* dst, const void* src, long long bytes, void* stream) {
  if (bytes < 0 || (bytes > 0 && (dst == nullptr || src == nullptr))) return 1;
  if (bytes == 0) return 0;
  return cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, STREAM(stream)) == cudaSuccess ? 0 : 5;
}

// ---- peer windows over CUDA IPC -------------------------------------------------------------------------------
// One dedicated device allocation per window, exported as a 64-byte handle that the other processes of the
// machine open to obtain a pointer they can load from and store to.  Used where the set of processes changes
// while the job runs (a fresh process can open the handles of processes that have been running for hours; the
// exchange itself travels through whatever the caller uses for small messages).
int fbam_ipc_alloc(void** out, long long bytes) {
  if (out == nullptr || bytes <= 0) return 1;
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) return 5;
  if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess) { cudaFree(p); return 5; }
  *out = p;
  return 0;
}
int fbam_ipc_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : 5; }
int fbam_ipc_export(void* p, unsigned char* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return 5;
  memcpy(handle64, &h, 64);
  return 0;
}
int fbam_ipc_open(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return 5;
  *out = p;
  return 0;
}
int fbam_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : 5; }

}  // extern "C"
