// Persistent recurrent LSTM kernels.
//
// The input projection X·W_ihᵀ for the whole sequence is one large tensor-core GEMM done elsewhere; what
// remains per time step is a (batch ≤ 8) x H · H x 4H product plus the gate arithmetic — far too small to
// launch as kernels 1024 times.  These kernels run the whole sequence in one cooperative launch:
//
//  * forward: CTA j owns 8 hidden units (32 gate rows of W_hh).  Its W_hh slice is loaded ONCE into
//    registers as mma.sync A-fragments (8 warps split K) and stays there for all T steps.  Per step
//    every warp multiplies its K-slice with h_{t-1} (read from a double-buffered global vector through
//    L2), partial sums are reduced through shared memory, 64 threads apply the gate non-linearities,
//    keep the cell state in registers, and publish the CTA's 8 new h values; one grid-wide barrier
//    (monotonic counter, bounded spin) separates steps.  The buffer of gate pre-activations is
//    overwritten in place with the activated gates, which is exactly what the backward pass needs.
//  * backward (BPTT): CTA j owns 16 hidden units: it keeps the matching 16 rows of W_hhᵀ (K = 4H) in
//    registers, does the point-wise gate gradient for its units, writes dGates[t] (bf16 — the big
//    dX / dW GEMMs consume it later), and after the barrier multiplies all of dGates[t] with its
//    W_hhᵀ rows to obtain dh_{t-1} for its own units, which never leaves the CTA.
//
// (The batch dimension is the 8-wide N of mma.sync.m16n8k16; the legacy tensor path is the right tool
// here: tcgen05 tiles start at M = 64 rows per CTA and would be ≥ 87 % padding for this shape.)
//
// The reference runs the recurrence as one GEMM launch plus a point-wise cell kernel per time step (reference:
// kernel_gen/kernel_gen/kernels/lstm_cell.py:6-144, kernels/lstm_cell_bwd.py:6-273 for the cell arithmetic and the
// recompute / backward point-wise kernels; tensorlib/src/streaming_lstm.cpp and streaming_lstm_bwd.cpp for the loop
// around them); gate order i, f, g, o, fp32 gates and cell state as there (tanh is tanhf here; the reference
// writes it as 2·sigmoid(2x) - 1, the same function).
#include <cooperative_groups.h>
#include "elem16.cuh"
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr unsigned kBarrierSpinLimit = 1u << 22;
enum { LSTM_ERR_BARRIER_TIMEOUT = 201 };

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs arrive; returns false (in every thread) if the wait ran out.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int* status) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    unsigned spins = 0;
    while (ld_acquire(counter) < target) {
      if (++spins > kBarrierSpinLimit) { ok = 0; break; }
      __nanosleep(20);
    }
    if (!ok) atomicExch(status, LSTM_ERR_BARRIER_TIMEOUT);
  }
  return __syncthreads_and(ok) != 0;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32." ELEM_PTX "." ELEM_PTX ".f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }

// -------------------------------------------------------------------------------------------------
// forward
// -------------------------------------------------------------------------------------------------
template <int MAXKS>  // k-steps (of 16) per warp: H <= MAXKS * 8 * 16
__global__ void __launch_bounds__(kThreads, 1)
lstm_fwd_kernel(float* __restrict__ gates, const elem_t* __restrict__ whh, const float* __restrict__ h0,
                const float* __restrict__ c0, elem_t* __restrict__ y, float* __restrict__ c_all, elem_t* hbuf,
                unsigned* counter, int* status, int T, int B, int H, int per_sample) {
  __shared__ float part[kWarps][2][16][8];
  __shared__ float pre[32][8];
  extern __shared__ uint4 dyn_smem[];
  elem_t* hs = reinterpret_cast<elem_t*>(dyn_smem);  // [8][H + 8]: h_{t-1}, rows padded by 16 B against bank conflicts
  const int hs_ld = H + 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int unit0 = blockIdx.x * 8;
  const int nks = H / 16;

  // W_hh slice -> registers (A fragments).  Tile 0 rows: gate i (0-7), gate f (8-15); tile 1: g, o.
  uint32_t afrag[2][MAXKS][4];
#pragma unroll
  for (int tile = 0; tile < 2; ++tile)
#pragma unroll
    for (int j = 0; j < MAXKS; ++j) {
      const int ks = warp + kWarps * j;
      const bool on = ks < nks;
      const int k = ks * 16 + q * 2;
      const elem_t* r_lo = whh + ((long long)(tile * 2) * H + unit0 + g) * H;      // row g   of the tile
      const elem_t* r_hi = whh + ((long long)(tile * 2 + 1) * H + unit0 + g) * H;  // row g+8 of the tile
      afrag[tile][j][0] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k) : 0u;
      afrag[tile][j][1] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k) : 0u;
      afrag[tile][j][2] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k + 8) : 0u;
      afrag[tile][j][3] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k + 8) : 0u;
    }

  // initial state: threads 0..63 own (unit u, batch b)
  const int u = threadIdx.x >> 3, b = threadIdx.x & 7;
  float c = 0.0f;
  if (threadIdx.x < 64) {
    // initial state: one learned vector broadcast over the batch, or (per_sample) a (B, H) state carried over
    // from the previous chunk of the same sequences
    const long long si = per_sample ? (long long)min(b, B - 1) * H + unit0 + u : unit0 + u;
    c = c0[si];
    hbuf[(long long)b * H + unit0 + u] = f2e(h0[si]);
  }
  // Each of the 256 threads owns one (gate row, batch) entry of the pre-activations; the value for the next
  // step is fetched from HBM before the grid barrier so that its latency is hidden behind the wait.
  const int prow = threadIdx.x >> 3, pbb = threadIdx.x & 7;
  const int ptile = prow >> 4, pr = prow & 15;
  const long long pre_off = (long long)(ptile * 2 + (pr >> 3)) * H + unit0 + (pr & 7);
  float xg_next = 0.0f;
  if (pbb < B) xg_next = gates[(long long)pbb * 4 * H + pre_off];
  unsigned bar = 0;
  if (!grid_barrier(counter, ++bar * gridDim.x, status)) return;

  for (int t = 0; t < T; ++t) {
    const float xg = xg_next;
    const elem_t* hprev = hbuf + (long long)(t & 1) * 8 * H;
    elem_t* hnext = hbuf + (long long)((t + 1) & 1) * 8 * H;
    // h_{t-1} (8 x H bf16) -> shared memory with independent 16-byte loads (one L2 round trip in flight
    // for all of them), then the B fragments come from shared memory.
    for (int c = threadIdx.x; c < H; c += kThreads) {  // 8*H/8 packets of 8 elements
      const int row = c / (H / 8), col = (c % (H / 8)) * 8;
      *reinterpret_cast<uint4*>(hs + row * hs_ld + col) =
          __ldcg(reinterpret_cast<const uint4*>(hprev + (long long)row * H + col));
    }
    __syncthreads();
    float acc[2][2][4] = {{{0, 0, 0, 0}, {0, 0, 0, 0}}, {{0, 0, 0, 0}, {0, 0, 0, 0}}};
#pragma unroll
    for (int j = 0; j < MAXKS; ++j) {
      const int ks = warp + kWarps * j;
      if (ks < nks) {
        const elem_t* hp = hs + g * hs_ld + ks * 16 + q * 2;  // B fragment: n = g (batch), k pairs
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(hp);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(hp + 8);
        mma_16816(acc[0][j & 1], afrag[0][j], b0, b1);
        mma_16816(acc[1][j & 1], afrag[1][j], b0, b1);
      }
    }
#pragma unroll
    for (int tile = 0; tile < 2; ++tile) {
      part[warp][tile][g][q * 2] = acc[tile][0][0] + acc[tile][1][0];
      part[warp][tile][g][q * 2 + 1] = acc[tile][0][1] + acc[tile][1][1];
      part[warp][tile][g + 8][q * 2] = acc[tile][0][2] + acc[tile][1][2];
      part[warp][tile][g + 8][q * 2 + 1] = acc[tile][0][3] + acc[tile][1][3];
    }
    __syncthreads();
    {
      const int row = threadIdx.x >> 3, bb = threadIdx.x & 7;  // 32 rows x 8 batch = 256 threads
      const int tile = row >> 4, r = row & 15;
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += part[w][tile][r][bb];
      pre[row][bb] = s + xg;
    }
    __syncthreads();
    if (threadIdx.x < 64) {
      const float ig = sigmoid_f(pre[u][b]), fg = sigmoid_f(pre[8 + u][b]);
      const float gg = tanhf(pre[16 + u][b]), og = sigmoid_f(pre[24 + u][b]);
      c = fg * c + ig * gg;
      const float h = og * tanhf(c);
      const elem_t hb = f2e(h);
      if (b < B) {
        float* gt = gates + ((long long)t * B + b) * 4 * H + unit0 + u;
        gt[0] = ig; gt[H] = fg; gt[2 * (long long)H] = gg; gt[3 * (long long)H] = og;
        y[((long long)t * B + b) * H + unit0 + u] = hb;
        c_all[((long long)t * B + b) * H + unit0 + u] = c;
        hnext[(long long)b * H + unit0 + u] = hb;
      } else {
        hnext[(long long)b * H + unit0 + u] = f2e(0.0f);
      }
    }
    // prefetch: the same thread wrote this location's activated gate for step t above only if it is one of
    // the 64 gate threads; the value read here belongs to step t+1, which nobody has touched yet.
    if (pbb < B && t + 1 < T) xg_next = gates[((long long)(t + 1) * B + pbb) * 4 * H + pre_off];
    if (!grid_barrier(counter, ++bar * gridDim.x, status)) return;
  }
}

// -------------------------------------------------------------------------------------------------
// backward
// -------------------------------------------------------------------------------------------------
template <int MAXKS>  // k-steps per warp: 4H <= MAXKS * 8 * 16
__global__ void __launch_bounds__(kThreads, 1)
lstm_bwd_kernel(const float* __restrict__ gates, const float* __restrict__ c_all, const float* __restrict__ c0,
                const elem_t* __restrict__ dy, const elem_t* __restrict__ whh_t, elem_t* dgates, float* __restrict__ dh0,
                float* __restrict__ dc0, const float* __restrict__ dh_last, const float* __restrict__ dc_last,
                unsigned* counter, int* status, int T, int B, int H, int per_sample) {
  __shared__ float part[kWarps][16][8];
  extern __shared__ uint4 dyn_smem[];
  elem_t* ds = reinterpret_cast<elem_t*>(dyn_smem);  // [8][4H + 8]: dGates[t], padded rows
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int unit0 = blockIdx.x * 16;
  const int K = 4 * H, nks = K / 16;
  const int ds_ld = K + 8;
  for (int c = threadIdx.x; c < 8 * ds_ld / 8; c += kThreads) dyn_smem[c] = make_uint4(0, 0, 0, 0);  // rows >= B stay 0

  uint32_t afrag[MAXKS][4];
#pragma unroll
  for (int j = 0; j < MAXKS; ++j) {
    const int ks = warp + kWarps * j;
    const bool on = ks < nks;
    const int k = ks * 16 + q * 2;
    const elem_t* r_lo = whh_t + (long long)(unit0 + g) * K;
    const elem_t* r_hi = whh_t + (long long)(unit0 + g + 8) * K;
    afrag[j][0] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k) : 0u;
    afrag[j][1] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k) : 0u;
    afrag[j][2] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k + 8) : 0u;
    afrag[j][3] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k + 8) : 0u;
  }

  const int u = threadIdx.x >> 3, b = threadIdx.x & 7;  // threads 0..127 own (unit u of 16, batch b)
  const bool owner = threadIdx.x < 128 && b < B;
  const int unit = unit0 + u;
  float dh_next = 0.0f, dc_next = 0.0f;
  if (owner) {
    if (dh_last != nullptr) dh_next = dh_last[(long long)b * H + unit];
    if (dc_last != nullptr) dc_next = dc_last[(long long)b * H + unit];
  }
  unsigned bar = 0;
  // point-wise inputs of the step about to be processed (fetched one step ahead, before the barrier)
  float n_ig = 0, n_fg = 0, n_gg = 0, n_og = 0, n_ct = 0, n_cp = 0, n_dy = 0;
  if (owner) {
    const int t = T - 1;
    const float* gt = gates + ((long long)t * B + b) * K + unit;
    n_ig = gt[0]; n_fg = gt[H]; n_gg = gt[2 * (long long)H]; n_og = gt[3 * (long long)H];
    n_ct = c_all[((long long)t * B + b) * H + unit];
    n_cp = t > 0 ? c_all[((long long)(t - 1) * B + b) * H + unit] : c0[per_sample ? (long long)b * H + unit : unit];
    n_dy = e2f(dy[((long long)t * B + b) * H + unit]);
  }

  for (int t = T - 1; t >= 0; --t) {
    if (owner) {
      const float ig = n_ig, fg = n_fg, gg = n_gg, og = n_og, ct = n_ct, cp = n_cp;
      const float dh = n_dy + dh_next;
      const float tc = tanhf(ct);
      const float d_o = dh * tc * og * (1.0f - og);
      const float dc = dh * og * (1.0f - tc * tc) + dc_next;
      const float d_i = dc * gg * ig * (1.0f - ig);
      const float d_f = dc * cp * fg * (1.0f - fg);
      const float d_g = dc * ig * (1.0f - gg * gg);
      dc_next = dc * fg;
      elem_t* dg = dgates + ((long long)t * B + b) * K + unit;
      dg[0] = f2e(d_i);
      dg[H] = f2e(d_f);
      dg[2 * (long long)H] = f2e(d_g);
      dg[3 * (long long)H] = f2e(d_o);
      if (t > 0) {
        const int tn = t - 1;
        const float* gt = gates + ((long long)tn * B + b) * K + unit;
        n_ig = gt[0]; n_fg = gt[H]; n_gg = gt[2 * (long long)H]; n_og = gt[3 * (long long)H];
        n_ct = cp;
        n_cp = tn > 0 ? c_all[((long long)(tn - 1) * B + b) * H + unit]
                      : c0[per_sample ? (long long)b * H + unit : unit];
        n_dy = e2f(dy[((long long)tn * B + b) * H + unit]);
      }
    }
    if (!grid_barrier(counter, ++bar * gridDim.x, status)) return;
    // dh_{t-1}[b, unit] = sum_k dGates[t][b, k] * W_hh[k, unit]
    const elem_t* dgt = dgates + (long long)t * B * K;
    for (int c = threadIdx.x; c < B * (K / 8); c += kThreads) {
      const int row = c / (K / 8), col = (c % (K / 8)) * 8;
      *reinterpret_cast<uint4*>(ds + row * ds_ld + col) =
          __ldcg(reinterpret_cast<const uint4*>(dgt + (long long)row * K + col));
    }
    __syncthreads();
    float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
    for (int j = 0; j < MAXKS; ++j) {
      const int ks = warp + kWarps * j;
      if (ks < nks) {
        const elem_t* p = ds + g * ds_ld + ks * 16 + q * 2;
        mma_16816(acc[j & 1], afrag[j], *reinterpret_cast<const uint32_t*>(p),
                  *reinterpret_cast<const uint32_t*>(p + 8));
      }
    }
    part[warp][g][q * 2] = acc[0][0] + acc[1][0];
    part[warp][g][q * 2 + 1] = acc[0][1] + acc[1][1];
    part[warp][g + 8][q * 2] = acc[0][2] + acc[1][2];
    part[warp][g + 8][q * 2 + 1] = acc[0][3] + acc[1][3];
    __syncthreads();
    if (threadIdx.x < 128) {
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += part[w][u][b];
      dh_next = s;
    }
    __syncthreads();
  }
  if (owner) {
    dh0[(long long)b * H + unit] = dh_next;
    dc0[(long long)b * H + unit] = dc_next;
  }
}

// -------------------------------------------------------------------------------------------------
// hidden sizes above 1024 (up to 2048): the W_hh slice of a CTA (256 KB at H = 2048) no longer fits in
// registers alone, so the kernels below run 16 warps and keep the first RKS k-steps of every warp in
// registers and the remaining SKS in shared memory, stored fragment by fragment (one conflict-free 16-byte
// read per thread and MMA).  Everything else follows the kernels above.
// -------------------------------------------------------------------------------------------------
constexpr int kBigWarps = 16;
constexpr int kBigThreads = kBigWarps * 32;

template <int RKS, int SKS>  // H <= (RKS + SKS) * 16 warps * 16
__global__ void __launch_bounds__(kBigThreads, 1)
lstm_fwd_big_kernel(float* __restrict__ gates, const elem_t* __restrict__ whh, const float* __restrict__ h0,
                    const float* __restrict__ c0, elem_t* __restrict__ y, float* __restrict__ c_all, elem_t* hbuf,
                    unsigned* counter, int* status, int T, int B, int H, int per_sample) {
  extern __shared__ uint4 dyn_smem[];
  uint4* wsm = dyn_smem;                                                  // [SKS * 4][512] A fragments
  elem_t* hs = reinterpret_cast<elem_t*>(dyn_smem + SKS * 4 * kBigThreads);   // [8][H + 8]
  const int hs_ld = H + 8;
  float* part = reinterpret_cast<float*>(hs + 8 * hs_ld);                 // [16 warps][4 tiles][16][8]
  float* pre = part + kBigWarps * 4 * 128;                                // [64][8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int unit0 = blockIdx.x * 16;  // 16 hidden units = 64 gate rows: tile = (unit group of 8) * 2 + {i|f, g|o}
  const int nks = H / 16;

  auto load_frag = [&](int tile, int ks, uint32_t (&a)[4]) {
    const bool on = ks < nks;
    const int k = ks * 16 + q * 2;
    const int unit = unit0 + (tile >> 1) * 8 + g;
    const elem_t* r_lo = whh + ((long long)((tile & 1) * 2) * H + unit) * H;
    const elem_t* r_hi = whh + ((long long)((tile & 1) * 2 + 1) * H + unit) * H;
    a[0] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k) : 0u;
    a[1] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k) : 0u;
    a[2] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k + 8) : 0u;
    a[3] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k + 8) : 0u;
  };
  uint32_t afrag[RKS][4][4];
#pragma unroll
  for (int j = 0; j < RKS; ++j)
#pragma unroll
    for (int tile = 0; tile < 4; ++tile) load_frag(tile, warp + kBigWarps * j, afrag[j][tile]);
#pragma unroll
  for (int j = 0; j < SKS; ++j)
#pragma unroll
    for (int tile = 0; tile < 4; ++tile) {
      uint32_t a[4];
      load_frag(tile, warp + kBigWarps * (RKS + j), a);
      wsm[(j * 4 + tile) * kBigThreads + threadIdx.x] = make_uint4(a[0], a[1], a[2], a[3]);
    }

  const int u = threadIdx.x >> 3, b = threadIdx.x & 7;  // threads 0..127 own (unit u of 16, batch b)
  float c = 0.0f;
  if (threadIdx.x < 128) {
    const long long si = per_sample ? (long long)min(b, B - 1) * H + unit0 + u : unit0 + u;
    c = c0[si];
    hbuf[(long long)b * H + unit0 + u] = f2e(h0[si]);
  }
  // every thread owns one (gate row of 64, batch) pre-activation, fetched one step ahead of its use
  const int prow = threadIdx.x >> 3, pbb = threadIdx.x & 7;
  const int ptile = prow >> 4, pr = prow & 15;
  const long long pre_off = (long long)((ptile & 1) * 2 + (pr >> 3)) * H + unit0 + (ptile >> 1) * 8 + (pr & 7);
  float xg_next = 0.0f;
  if (pbb < B) xg_next = gates[(long long)pbb * 4 * H + pre_off];
  unsigned bar = 0;
  if (!grid_barrier(counter, ++bar * gridDim.x, status)) return;

  for (int t = 0; t < T; ++t) {
    const float xg = xg_next;
    const elem_t* hprev = hbuf + (long long)(t & 1) * 8 * H;
    elem_t* hnext = hbuf + (long long)((t + 1) & 1) * 8 * H;
    for (int cc = threadIdx.x; cc < H; cc += kBigThreads) {
      const int row = cc / (H / 8), col = (cc % (H / 8)) * 8;
      *reinterpret_cast<uint4*>(hs + row * hs_ld + col) =
          __ldcg(reinterpret_cast<const uint4*>(hprev + (long long)row * H + col));
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int tile = 0; tile < 4; ++tile)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[tile][i] = 0.0f;
#pragma unroll
    for (int j = 0; j < RKS + SKS; ++j) {
      const int ks = warp + kBigWarps * j;
      if (ks < nks) {
        const elem_t* hp = hs + g * hs_ld + ks * 16 + q * 2;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(hp);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(hp + 8);
#pragma unroll
        for (int tile = 0; tile < 4; ++tile) {
          if (j < RKS) {
            mma_16816(acc[tile], afrag[j < RKS ? j : 0][tile], b0, b1);
          } else {
            const uint4 w = wsm[((j - RKS) * 4 + tile) * kBigThreads + threadIdx.x];
            const uint32_t a[4] = {w.x, w.y, w.z, w.w};
            mma_16816(acc[tile], a, b0, b1);
          }
        }
      }
    }
#pragma unroll
    for (int tile = 0; tile < 4; ++tile) {
      float* pt = part + (warp * 4 + tile) * 128;
      pt[g * 8 + q * 2] = acc[tile][0];
      pt[g * 8 + q * 2 + 1] = acc[tile][1];
      pt[(g + 8) * 8 + q * 2] = acc[tile][2];
      pt[(g + 8) * 8 + q * 2 + 1] = acc[tile][3];
    }
    __syncthreads();
    {
      float s = 0.0f;  // thread = (row of 64, batch): row = tile * 16 + r
#pragma unroll
      for (int w = 0; w < kBigWarps; ++w) s += part[(w * 4 + ptile) * 128 + pr * 8 + pbb];
      pre[prow * 8 + pbb] = s + xg;
    }
    __syncthreads();
    if (threadIdx.x < 128) {
      const int base = (u >> 3) * 32 + (u & 7);  // tile pair of the unit group; rows +0 i, +8 f, +16 g, +24 o
      const float ig = sigmoid_f(pre[base * 8 + b]), fg = sigmoid_f(pre[(base + 8) * 8 + b]);
      const float gg = tanhf(pre[(base + 16) * 8 + b]), og = sigmoid_f(pre[(base + 24) * 8 + b]);
      c = fg * c + ig * gg;
      const float h = og * tanhf(c);
      const elem_t hb = f2e(h);
      if (b < B) {
        float* gt = gates + ((long long)t * B + b) * 4 * H + unit0 + u;
        gt[0] = ig; gt[H] = fg; gt[2 * (long long)H] = gg; gt[3 * (long long)H] = og;
        y[((long long)t * B + b) * H + unit0 + u] = hb;
        c_all[((long long)t * B + b) * H + unit0 + u] = c;
        hnext[(long long)b * H + unit0 + u] = hb;
      } else {
        hnext[(long long)b * H + unit0 + u] = f2e(0.0f);
      }
    }
    if (pbb < B && t + 1 < T) xg_next = gates[((long long)(t + 1) * B + pbb) * 4 * H + pre_off];
    if (!grid_barrier(counter, ++bar * gridDim.x, status)) return;
  }
}

// Backward: the CTA's 16 rows of W_hh^T span K = 4H (8192 at H = 2048).  dGates[t] is staged in two halves of K
// so that the staging buffer and the shared-memory part of the weights fit together; the first half's k-steps
// use the register fragments, the second half's the shared-memory ones.
template <int HKS>  // k-steps per warp and half: 4H <= 2 * HKS * 16 warps * 16
__global__ void __launch_bounds__(kBigThreads, 1)
lstm_bwd_big_kernel(const float* __restrict__ gates, const float* __restrict__ c_all, const float* __restrict__ c0,
                    const elem_t* __restrict__ dy, const elem_t* __restrict__ whh_t, elem_t* dgates,
                    float* __restrict__ dh0, float* __restrict__ dc0, const float* __restrict__ dh_last,
                    const float* __restrict__ dc_last, unsigned* counter, int* status, int T, int B, int H,
                    int per_sample) {
  extern __shared__ uint4 dyn_smem[];
  uint4* wsm = dyn_smem;                                              // [HKS][512] A fragments (second half of K)
  elem_t* ds = reinterpret_cast<elem_t*>(dyn_smem + HKS * kBigThreads);   // [8][K/2 + 8]: half of dGates[t]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int unit0 = blockIdx.x * 16;
  const int K = 4 * H, kh = K / 32;  // k-steps per half
  const int ds_ld = K / 2 + 8;
  float* part = reinterpret_cast<float*>(ds + 8 * ds_ld);             // [16 warps][16][8]
  for (int cc = threadIdx.x; cc < 8 * ds_ld / 8; cc += kBigThreads)   // rows >= B stay zero
    reinterpret_cast<uint4*>(ds)[cc] = make_uint4(0, 0, 0, 0);

  auto load_frag = [&](int ks, bool on, uint32_t (&a)[4]) {
    const int k = ks * 16 + q * 2;
    const elem_t* r_lo = whh_t + (long long)(unit0 + g) * K;
    const elem_t* r_hi = whh_t + (long long)(unit0 + g + 8) * K;
    a[0] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k) : 0u;
    a[1] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k) : 0u;
    a[2] = on ? *reinterpret_cast<const uint32_t*>(r_lo + k + 8) : 0u;
    a[3] = on ? *reinterpret_cast<const uint32_t*>(r_hi + k + 8) : 0u;
  };
  uint32_t afrag[HKS][4];
#pragma unroll
  for (int j = 0; j < HKS; ++j) {
    const int ks = warp + kBigWarps * j;
    load_frag(ks, ks < kh, afrag[j]);
    uint32_t a[4];
    load_frag(kh + ks, ks < kh, a);
    wsm[j * kBigThreads + threadIdx.x] = make_uint4(a[0], a[1], a[2], a[3]);
  }

  const int u = threadIdx.x >> 3, b = threadIdx.x & 7;
  const bool owner = threadIdx.x < 128 && b < B;
  const int unit = unit0 + (u & 15);
  float dh_next = 0.0f, dc_next = 0.0f;
  if (owner) {
    if (dh_last != nullptr) dh_next = dh_last[(long long)b * H + unit];
    if (dc_last != nullptr) dc_next = dc_last[(long long)b * H + unit];
  }
  unsigned bar = 0;
  float n_ig = 0, n_fg = 0, n_gg = 0, n_og = 0, n_ct = 0, n_cp = 0, n_dy = 0;
  if (owner) {
    const int t = T - 1;
    const float* gt = gates + ((long long)t * B + b) * K + unit;
    n_ig = gt[0]; n_fg = gt[H]; n_gg = gt[2 * (long long)H]; n_og = gt[3 * (long long)H];
    n_ct = c_all[((long long)t * B + b) * H + unit];
    n_cp = t > 0 ? c_all[((long long)(t - 1) * B + b) * H + unit] : c0[per_sample ? (long long)b * H + unit : unit];
    n_dy = e2f(dy[((long long)t * B + b) * H + unit]);
  }

  for (int t = T - 1; t >= 0; --t) {
    if (owner) {
      const float ig = n_ig, fg = n_fg, gg = n_gg, og = n_og, ct = n_ct, cp = n_cp;
      const float dh = n_dy + dh_next;
      const float tc = tanhf(ct);
      const float d_o = dh * tc * og * (1.0f - og);
      const float dc = dh * og * (1.0f - tc * tc) + dc_next;
      const float d_i = dc * gg * ig * (1.0f - ig);
      const float d_f = dc * cp * fg * (1.0f - fg);
      const float d_g = dc * ig * (1.0f - gg * gg);
      dc_next = dc * fg;
      elem_t* dg = dgates + ((long long)t * B + b) * K + unit;
      dg[0] = f2e(d_i);
      dg[H] = f2e(d_f);
      dg[2 * (long long)H] = f2e(d_g);
      dg[3 * (long long)H] = f2e(d_o);
      if (t > 0) {
        const int tn = t - 1;
        const float* gt = gates + ((long long)tn * B + b) * K + unit;
        n_ig = gt[0]; n_fg = gt[H]; n_gg = gt[2 * (long long)H]; n_og = gt[3 * (long long)H];
        n_ct = cp;
        n_cp = tn > 0 ? c_all[((long long)(tn - 1) * B + b) * H + unit]
                      : c0[per_sample ? (long long)b * H + unit : unit];
        n_dy = e2f(dy[((long long)tn * B + b) * H + unit]);
      }
    }
    if (!grid_barrier(counter, ++bar * gridDim.x, status)) return;
    const elem_t* dgt = dgates + (long long)t * B * K;
    float acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int hcols = K / 2;
      for (int cc = threadIdx.x; cc < B * (hcols / 8); cc += kBigThreads) {
        const int row = cc / (hcols / 8), col = (cc % (hcols / 8)) * 8;
        *reinterpret_cast<uint4*>(ds + row * ds_ld + col) =
            __ldcg(reinterpret_cast<const uint4*>(dgt + (long long)row * K + half * hcols + col));
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < HKS; ++j) {
        const int ks = warp + kBigWarps * j;
        if (ks < kh) {
          const elem_t* p = ds + g * ds_ld + ks * 16 + q * 2;
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(p), b1 = *reinterpret_cast<const uint32_t*>(p + 8);
          if (half == 0) {
            mma_16816(acc[j & 1], afrag[j], b0, b1);
          } else {
            const uint4 w = wsm[j * kBigThreads + threadIdx.x];
            const uint32_t a[4] = {w.x, w.y, w.z, w.w};
            mma_16816(acc[j & 1], a, b0, b1);
          }
        }
      }
      __syncthreads();
    }
    float* pt = part + warp * 128;
    pt[g * 8 + q * 2] = acc[0][0] + acc[1][0];
    pt[g * 8 + q * 2 + 1] = acc[0][1] + acc[1][1];
    pt[(g + 8) * 8 + q * 2] = acc[0][2] + acc[1][2];
    pt[(g + 8) * 8 + q * 2 + 1] = acc[0][3] + acc[1][3];
    __syncthreads();
    if (threadIdx.x < 128) {
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < kBigWarps; ++w) s += part[w * 128 + u * 8 + b];
      dh_next = s;
    }
    __syncthreads();
  }
  if (owner) {
    dh0[(long long)b * H + unit] = dh_next;
    dc0[(long long)b * H + unit] = dc_next;
  }
}

template <typename K>
int coop_launch(K kernel, int grid, void** args, size_t smem, cudaStream_t stream, int threads = kThreads) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return 5;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) return 5;
  if (grid > sms * per_sm) return 1;  // all CTAs must be co-resident
  return cudaLaunchCooperativeKernel((void*)kernel, dim3(grid), dim3(threads), args, smem, stream) == cudaSuccess
             ? 0 : 5;
}

}  // namespace

extern "C" {

// Largest hidden size the register-resident kernels accept (and the batch limit is 8).
int fbam_lstm_persistent_max_hidden() { return 2048; }

// gates: (T, B, 4H) fp32, pre-activations incl. bias on entry, activated gates on exit.
// hbuf: 2*8*H bf16 scratch; counter: one zeroed unsigned.
int fbam_lstm_fwd_ex(float* gates, const void* whh, const float* h0, const float* c0, void* y, float* c_all,
                     void* hbuf, unsigned* counter, int* status, int T, int B, int H, int per_sample, void* stream) {
  if (B < 1 || B > 8 || H % 16 != 0 || H > 2048 || T < 1) return 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(counter, 0, sizeof(unsigned), s) != cudaSuccess) return 5;
  void* args[] = {&gates, &whh, &h0, &c0, &y, &c_all, &hbuf, &counter, &status, &T, &B, &H, &per_sample};
  if (H > 1024) {  // 16 units per CTA; half of each warp's 8 k-steps in registers, half in shared memory
    const size_t big = (size_t)4 * 4 * kBigThreads * 16 + (size_t)8 * (H + 8) * sizeof(elem_t) +
                       (size_t)(kBigWarps * 4 * 128 + 64 * 8) * sizeof(float);
    return coop_launch(lstm_fwd_big_kernel<4, 4>, H / 16, args, big, s, kBigThreads);
  }
  const int grid = H / 8;
  const size_t smem = (size_t)8 * (H + 8) * sizeof(elem_t);
  if (H <= 256) return coop_launch(lstm_fwd_kernel<2>, grid, args, smem, s);
  if (H <= 512) return coop_launch(lstm_fwd_kernel<4>, grid, args, smem, s);
  return coop_launch(lstm_fwd_kernel<8>, grid, args, smem, s);
}

// h0 / c0 are (H) vectors broadcast over the batch.
int fbam_lstm_fwd(float* gates, const void* whh, const float* h0, const float* c0, void* y, float* c_all,
                  void* hbuf, unsigned* counter, int* status, int T, int B, int H, void* stream) {
  return fbam_lstm_fwd_ex(gates, whh, h0, c0, y, c_all, hbuf, counter, status, T, B, H, 0, stream);
}

// whh_t: (H, 4H) bf16 = W_hh transposed.  dgates: (T, B, 4H) bf16 out.  dh0/dc0: (B, H) fp32 out.
int fbam_lstm_bwd_ex(const float* gates, const float* c_all, const float* c0, const void* dy, const void* whh_t,
                     void* dgates, float* dh0, float* dc0, const float* dh_last, const float* dc_last,
                     unsigned* counter, int* status, int T, int B, int H, int per_sample, void* stream) {
  if (B < 1 || B > 8 || H % 16 != 0 || H > 2048 || T < 1) return 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(counter, 0, sizeof(unsigned), s) != cudaSuccess) return 5;
  void* args[] = {&gates, &c_all, &c0, &dy, &whh_t, &dgates, &dh0, &dc0, &dh_last, &dc_last, &counter, &status,
                  &T, &B, &H, &per_sample};
  if (H > 1024) {
    const size_t big = (size_t)16 * kBigThreads * 16 + (size_t)8 * (2 * H + 8) * sizeof(elem_t) +
                       (size_t)kBigWarps * 128 * sizeof(float);
    return coop_launch(lstm_bwd_big_kernel<16>, H / 16, args, big, s, kBigThreads);
  }
  const int grid = H / 16;
  const size_t smem = (size_t)8 * (4 * H + 8) * sizeof(elem_t);
  if (H <= 256) return coop_launch(lstm_bwd_kernel<8>, grid, args, smem, s);
  if (H <= 512) return coop_launch(lstm_bwd_kernel<16>, grid, args, smem, s);
  return coop_launch(lstm_bwd_kernel<32>, grid, args, smem, s);
}

int fbam_lstm_bwd(const float* gates, const float* c_all, const float* c0, const void* dy, const void* whh_t,
                  void* dgates, float* dh0, float* dc0, const float* dh_last, const float* dc_last, unsigned* counter,
                  int* status, int T, int B, int H, void* stream) {
  return fbam_lstm_bwd_ex(gates, c_all, c0, dy, whh_t, dgates, dh0, dc0, dh_last, dc_last, counter, status, T, B, H, 0,
                          stream);
}

}  // extern "C"

// -------------------------------------------------------------------------------------------------
// Allocation-free variant of the forward entry point (see lstm_noalloc.h for who needs it and the contract).
// The scratch lives in a device array that is part of this module: [0, 256) holds the grid-barrier counter,
// the rest the double-buffered h vector for the largest supported hidden size.
// -------------------------------------------------------------------------------------------------
#include "lstm_noalloc.h"

#include <atomic>

static __device__ __align__(256) unsigned char g_lstm_noalloc_scratch[FBAM_LSTM_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
// Device address of the scratch array per device ordinal.  In host code the array's name is only a handle for
// the runtime; the address a kernel can use has to be asked for, once per device, with that device current.
// Atomic slots: two host threads making their first call on a device may both look the address up; they store the
// same value, and the atomics make that a defined race-free publication.
std::atomic<void*> g_noalloc_scratch_addr[kMaxDevices];

int noalloc_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FBAM_LSTM_NOALLOC_ERR_SETUP;
  void* ptr = g_noalloc_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    if (cudaGetSymbolAddress(&ptr, g_lstm_noalloc_scratch) != cudaSuccess || ptr == nullptr)
      return FBAM_LSTM_NOALLOC_ERR_SETUP;
    g_noalloc_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return 0;
}
}  // namespace

extern "C" {

int fbam_lstm_fwd_noalloc_max_hidden(void) { return FBAM_LSTM_NOALLOC_MAX_HIDDEN; }

const char* fbam_lstm_fwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case 1: return "unsupported shape: need 1 <= B <= 8, H a multiple of 16, T >= 1";
    case 5: return "kernel launch failed";
    case FBAM_LSTM_NOALLOC_ERR_TOO_LARGE:
      return "hidden size exceeds FBAM_LSTM_NOALLOC_MAX_HIDDEN (1024): the built-in scratch array is too small; "
             "use fbam_lstm_fwd with caller-provided scratch instead";
    case FBAM_LSTM_NOALLOC_ERR_SETUP: return "could not obtain the device address of the built-in scratch array";
    default: return "unknown error";
  }
}

int fbam_lstm_fwd_noalloc(float* gates, const void* whh, const float* h0, const float* c0, void* y, float* c_all,
                          int* status, int T, int B, int H, void* stream) {
  if (H > FBAM_LSTM_NOALLOC_MAX_HIDDEN) return FBAM_LSTM_NOALLOC_ERR_TOO_LARGE;
  if (B < 1 || B > 8 || H < 16 || H % 16 != 0 || T < 1) return 1;
  void* base = nullptr;
  const int rc = noalloc_scratch(&base);
  if (rc != 0) return rc;
  unsigned* counter = reinterpret_cast<unsigned*>(base);
  void* hbuf = static_cast<unsigned char*>(base) + 256;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the counter must start at zero; the h buffer is written (initial state) before any CTA reads it
  if (cudaMemsetAsync(counter, 0, sizeof(unsigned), s) != cudaSuccess) return 5;
  int per_sample = 0;
  void* args[] = {&gates, &whh, &h0, &c0, &y, &c_all, &hbuf, &counter, &status, &T, &B, &H, &per_sample};
  const int grid = H / 8;
  const size_t smem = (size_t)8 * (H + 8) * sizeof(elem_t);
  if (H <= 256) return coop_launch(lstm_fwd_kernel<2>, grid, args, smem, s);
  if (H <= 512) return coop_launch(lstm_fwd_kernel<4>, grid, args, smem, s);
  return coop_launch(lstm_fwd_kernel<8>, grid, args, smem, s);
}

}  // extern "C"
