// Flash-style multi-head attention for sm_100a on tcgen05 tensor cores (causal and non-causal, head
// dimension 64 or 128, bf16, fp32 softmax statistics).
//
// Forward: one CTA per (batch, head, block of 128 queries).  Q stays in shared memory; K/V blocks of 128
// keys stream through a two-stage TMA ring.  Per key block:  S = Q·Kᵀ is a tcgen05.mma into TMEM; the 128
// softmax threads — one query row each, so row max / row sum need no shuffles — read S with tcgen05.ld,
// write P = exp2(scale·S − m) as bf16 into shared memory in the 128-byte-swizzled K-major layout, and the
// second tcgen05.mma computes P·V into TMEM with V consumed in place as an MN-major operand (keys are its K
// dimension, so no transposed copy of V exists).  The running output lives in registers:
// O ← O·exp2(m_old − m_new) + P·V.  The log-sum-exp per row is stored for the backward pass.
//
// Backward: one CTA per (batch, head, block of 128 keys) walks the query blocks that attend to it and, per
// block, issues five tcgen05 GEMMs: S = Q·Kᵀ and dP = dO·Vᵀ into TMEM, then — after the 128 threads rebuilt
// P = exp2(scale·S − lse) and dS = P∘(dP − δ) in shared memory — dV += Pᵀ·dO, dK += dSᵀ·Q (accumulating in
// TMEM across query blocks; P and dS are read as MN-major A operands, i.e. transposed for free) and
// dQ_block = dS·K, which is added into an fp32 dQ buffer with atomics.  δ = rowsum(dO∘O) comes from a small
// pre-pass kernel.
//
// Q/K/V/O/dO are addressed as (B, T, H, D) views with arbitrary batch / row / head strides (the fused QKV
// projection output is used in place).  All mbarrier waits are bounded.
//
// Takes the place of the reference's attention kernels: flash-attention forward with log-sum-exp output, the
// dO·O pre-pass and the backward producing dQ, dK, dV (reference:
// kernel_gen/kernel_gen/kernels/flash_attention_codegen/compile.py:280-330, kernels/flash_attention_fwd.py:36-266,
// kernels/flash_attention_bwd.py:6-313; selected in src/passes/mha_attention_pass.cpp).  The reference supports
// head dimension 128 only; 64 is added here.
#include "tc05.cuh"

namespace {

using namespace tc05;

constexpr int BQ = 128;   // queries per tile (TMEM lanes)
constexpr int BKV = 128;  // keys per block
enum { ATT_ERR_TIMEOUT = 501 };

struct AttnParams {
  int B, T, H, D;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  float scale;
  elem_t* out;         // (B, T, H, D) contiguous
  float* lse;        // (B, H, T), natural-log units of the scaled scores
  int* status;
};

__device__ __forceinline__ void tma_load_attn(void* dst, const CUtensorMap* map, uint64_t* bar, int d0, int h, int t,
                                              int b) {
  tma_load_4d(dst, map, bar, d0, h, t, b);
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Address of element (row, col8 = 8-element group index) in a [rows x 64]-bf16 panel with 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// -------------------------------------------------------------------------------------------------
// forward
// -------------------------------------------------------------------------------------------------
// KV_STAGES = 2 prefetches the next K/V block inside the CTA; KV_STAGES = 1 halves the K/V footprint so that two
// CTAs share an SM and overlap each other's softmax and tensor-core phases instead (used for D = 64).
template <int D, int KV_STAGES>
__global__ void __launch_bounds__(160, KV_STAGES == 1 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  constexpr int DP = D / 64;                 // 64-wide panels per row
  constexpr int kQBytes = BQ * D * 2;
  constexpr int kKVBytes = BKV * D * 2;
  constexpr int kPBytes = BQ * BKV * 2;
  constexpr uint32_t kTmemCols = 256;        // S: [0,128)  PV: [128, 128 + D)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;                // KV_STAGES stages
  uint8_t* sV = sK + KV_STAGES * kKVBytes;   // KV_STAGES stages
  uint8_t* sP = sV + KV_STAGES * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kPBytes);
  uint64_t* q_full = bars;                   // 1
  uint64_t* kv_full = bars + 1;              // 2
  uint64_t* kv_empty = bars + 3;             // 2
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* pv_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb * BQ;
  const int nkb = p.causal ? min((p.T + BKV - 1) / BKV, qb + 1) : (p.T + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(pv_full, 1);
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s = tmem, tmem_pv = tmem + 128;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      // Q once; first K/V block
      mbar_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int j = 0; j < DP; ++j) tma_load_attn(sQ + j * BQ * 128, &map_q, q_full, j * 64, h, q0, b);
      auto load_kv = [&](int kb) {
        const int s = kb % KV_STAGES;
        mbar_expect_tx(&kv_full[s], 2 * kKVBytes);
#pragma unroll
        for (int j = 0; j < DP; ++j) {
          tma_load_attn(sK + s * kKVBytes + j * BKV * 128, &map_k, &kv_full[s], j * 64, h, kb * BKV, b);
          tma_load_attn(sV + s * kKVBytes + j * BKV * 128, &map_v, &kv_full[s], j * 64, h, kb * BKV, b);
        }
      };
      load_kv(0);
      const uint32_t idesc_s = make_idesc_f16kind(128, BKV, false, false);
      const uint32_t idesc_pv = make_idesc_f16kind(128, D, false, true);   // B = V is MN-major
      ok = mbar_wait(q_full, 0);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % KV_STAGES;
        if (KV_STAGES == 2 && kb + 1 < nkb) {   // prefetch the next block into the other stage once it is free
          if (kb >= 1 && !mbar_wait(&kv_empty[s ^ 1], ((kb - 1) >> 1) & 1)) { ok = false; break; }
          load_kv(kb + 1);
        }
        if (KV_STAGES == 1 && kb >= 1) {        // single stage: reload once the previous block's P·V has read it
          if (!mbar_wait(&kv_empty[0], (kb - 1) & 1)) { ok = false; break; }
          load_kv(kb);
        }
        if (!mbar_wait(&kv_full[s], (kb / KV_STAGES) & 1)) { ok = false; break; }
        fence_after_sync();
        const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK + s * kKVBytes), v_addr = smem_u32(sV + s * kKVBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {   // K-major operands: panel k/4, 32 bytes per step inside the panel
          const uint64_t da = make_smem_desc_sw128(q_addr + (k / 4) * BQ * 128 + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(k_addr + (k / 4) * BKV * 128 + (k % 4) * 32, 16, 1024);
          mma_f16_ss(tmem_s, da, db, idesc_s, k != 0);
        }
        mma_commit(s_full);
        if (!mbar_wait(p_ready, kb & 1)) { ok = false; break; }
        fence_after_sync();
        const uint32_t p_addr = smem_u32(sP);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // A = P, K-major over keys: two 64-key panels.  B = V, MN-major: 16 key rows per step = 2048 bytes;
          // 64-wide D panels are BKV*128 bytes apart (leading-dimension offset).
          const uint64_t da = make_smem_desc_sw128(p_addr + (k / 4) * BQ * 128 + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(v_addr + k * 16 * 128, BKV * 128, 1024);
          mma_f16_ss(tmem_pv, da, db, idesc_pv, k != 0);
        }
        mma_commit(pv_full);
        mma_commit(&kv_empty[s]);
      }
      if (!ok) atomicExch(p.status, ATT_ERR_TIMEOUT);
    }
  } else {
    // ---------------------------------------------------------------- softmax / output threads
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;          // query row within the tile == TMEM lane
    const int t_q = q0 + row;
    const uint32_t lane_addr = uint32_t(lane_group * 32) << 16;
    float m = -INFINITY, l = 0.0f;
    float o[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o[d] = 0.0f;
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      if (!mbar_wait(s_full, kb & 1)) { ok = false; break; }
      fence_after_sync();
      const int k0 = kb * BKV;
      const bool need_mask = (p.causal && kb == qb) || (k0 + BKV > p.T);
      // pass 1: row maximum
      float mx = m;
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_s + lane_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float sv = __uint_as_float(r[j]);
          if (need_mask) {
            const int tk = k0 + c0 + j;
            if (tk >= p.T || (p.causal && tk > t_q)) sv = -INFINITY;
          }
          mx = fmaxf(mx, sv);
        }
      }
      const float m_new = mx;
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;   // fully masked row: keep exponents finite
      const float alpha = fast_exp2((m - m_use) * p.scale_log2);     // m = -inf on the first block -> 0
      float rs = 0.0f;
      // pass 2: P = exp2(scale*(S - m)) -> bf16 -> swizzled shared memory
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_s + lane_addr + c0, r);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float sv = __uint_as_float(r[j]);
          if (need_mask) {
            const int tk = k0 + c0 + j;
            if (tk >= p.T || (p.causal && tk > t_q)) sv = -INFINITY;
          }
          pv[j] = fast_exp2((sv - m_use) * p.scale_log2);
        }
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          __align__(16) elem2_t hh[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            hh[q] = ff2e2(pv[j8 * 8 + 2 * q], pv[j8 * 8 + 2 * q + 1]);
            const float2 back = e22ff(hh[q]);   // sum what the tensor core will actually see
            rs += back.x + back.y;
          }
          const int chunk = (c0 >> 3) + j8;                  // 16-byte chunk index within the 128-key row
          uint8_t* dst = sP + (chunk >> 3) * BQ * 128 + swz(row, chunk & 7);
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(hh);
        }
      }
      l = l * alpha + rs;
      m = m_new;
      fence_proxy_async();
      fence_before_sync();
      mbar_arrive(p_ready);
      // accumulate P·V
      if (!mbar_wait(pv_full, kb & 1)) { ok = false; break; }
      fence_after_sync();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_pv + lane_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) o[c0 + j] = o[c0 + j] * alpha + __uint_as_float(r[j]);
      }
      fence_before_sync();
    }
    if (ok && t_q < p.T) {
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      elem_t* dst = p.out + (((long long)b * p.T + t_q) * p.H + h) * D;
#pragma unroll
      for (int d = 0; d < D; d += 8) {
        __align__(16) elem2_t hh[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) hh[q] = ff2e2(o[d + 2 * q] * inv, o[d + 2 * q + 1] * inv);
        *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<uint4*>(hh);
      }
      if (p.lse != nullptr)
        p.lse[((long long)b * p.H + h) * p.T + t_q] = (l > 0.0f) ? m * p.scale + logf(l) : -INFINITY;
    }
    if (!ok && lane == 0) atomicExch(p.status, ATT_ERR_TIMEOUT);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc(tmem, kTmemCols); }
}

// -------------------------------------------------------------------------------------------------
// forward, two query tiles per CTA
// -------------------------------------------------------------------------------------------------
// Same arithmetic as attn_fwd_kernel, organised for more softmax throughput per SM: a CTA owns 256 consecutive
// queries of one head as two 128-row tiles, each with its own group of four softmax warps, its own S and P·V
// accumulators in TMEM (S_A, S_B, O_A, O_B = 256 + 2·D columns) and its own P buffer in shared memory; K and V
// blocks (one stage each, loaded as soon as the MMAs that read the previous block have completed) are shared by
// both tiles.  One elected thread issues all TMA loads and all MMAs in an order in which no tile ever waits for
// the other: while one group is busy with its softmax, the tensor core works for the other one.  The output
// accumulators stay in tensor memory for the whole key loop (every P·V product adds to them); the softmax threads
// rescale them there only when a row's reference maximum moves (see below), so a group goes from one block's softmax
// straight to the next while its P·V product is still running.
template <int D>
__global__ void __launch_bounds__(288, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  constexpr int DP = D / 64;
  constexpr int kQBytes = BQ * D * 2;      // one query tile
  constexpr int kKVBytes = BKV * D * 2;
  constexpr int kPBytes = BQ * BKV * 2;
  constexpr uint32_t kTmemCols = 512;      // S_A [0,128) S_B [128,256) O_A [256,256+D) O_B [256+D,256+2D)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // two tiles
  uint8_t* sK = sQ + 2 * kQBytes;
  uint8_t* sV = sK + kKVBytes;
  uint8_t* sP = sV + kKVBytes;             // two tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPBytes);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;             // [2]
  uint64_t* p_ready = bars + 7;            // [2]
  uint64_t* pv_full = bars + 9;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal: the tiles with the most key blocks are scheduled first
  const int qb2 = p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = qb2 * 2 * BQ;
  const int nkb_all = (p.T + BKV - 1) / BKV;
  // key blocks each tile attends to (a tile that starts beyond the sequence has none)
  int nkb_tile[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int qb = qb2 * 2 + g;
    nkb_tile[g] = (q0 + g * BQ >= p.T) ? 0 : (p.causal ? min(nkb_all, qb + 1) : nkb_all);
  }
  const int nkb = max(nkb_tile[0], nkb_tile[1]);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    for (int g = 0; g < 2; ++g) {
      mbar_init(&s_full[g], 1);
      mbar_init(&p_ready[g], 128);
      mbar_init(&pv_full[g], 1);
    }
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      mbar_expect_tx(q_full, 2 * kQBytes);
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int j = 0; j < DP; ++j)   // rows beyond the sequence are filled with zeros by TMA
          tma_load_attn(sQ + g * kQBytes + j * BQ * 128, &map_q, q_full, j * 64, h, q0 + g * BQ, b);
      auto load_k = [&](int kb) {
        mbar_expect_tx(k_full, kKVBytes);
#pragma unroll
        for (int j = 0; j < DP; ++j) tma_load_attn(sK + j * BKV * 128, &map_k, k_full, j * 64, h, kb * BKV, b);
      };
      auto load_v = [&](int kb) {
        mbar_expect_tx(v_full, kKVBytes);
#pragma unroll
        for (int j = 0; j < DP; ++j) tma_load_attn(sV + j * BKV * 128, &map_v, v_full, j * 64, h, kb * BKV, b);
      };
      const uint32_t idesc_s = make_idesc_f16kind(128, BKV, false, false);
      const uint32_t idesc_pv = make_idesc_f16kind(128, D, false, true);   // B = V is MN-major
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      auto issue_s = [&](int g) {      // S_g = Q_g · Kᵀ
        const uint32_t q_addr = smem_u32(sQ + g * kQBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(q_addr + (k / 4) * BQ * 128 + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(k_addr + (k / 4) * BKV * 128 + (k % 4) * 32, 16, 1024);
          mma_f16_ss(tmem + g * 128, da, db, idesc_s, k != 0);
        }
        mma_commit(&s_full[g]);
      };
      auto issue_pv = [&](int g, bool first) {     // O_g (+)= P_g · V: accumulated over the key blocks in tensor memory
        const uint32_t p_addr = smem_u32(sP + g * kPBytes);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(p_addr + (k / 4) * BQ * 128 + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(v_addr + k * 16 * 128, BKV * 128, 1024);
          mma_f16_ss(tmem + 256 + g * D, da, db, idesc_pv, !first || k != 0);
        }
        mma_commit(&pv_full[g]);
      };
      if (nkb > 0) {
        load_k(0);
        load_v(0);
        ok = mbar_wait(q_full, 0) && mbar_wait(k_full, 0);
        if (ok) {
          fence_after_sync();
          if (0 < nkb_tile[0]) issue_s(0);
          if (0 < nkb_tile[1]) issue_s(1);
          mma_commit(k_empty);
        }
      }
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const uint32_t ph = kb & 1;
        const bool more = kb + 1 < nkb;
        if (more) {                          // K block kb has been read by both S MMAs: fetch the next one
          if (!mbar_wait(k_empty, ph)) { ok = false; break; }
          load_k(kb + 1);
        }
        if (!mbar_wait(v_full, ph)) { ok = false; break; }
        if (kb < nkb_tile[0]) {
          if (!mbar_wait(&p_ready[0], ph)) { ok = false; break; }
          fence_after_sync();
          issue_pv(0, kb == 0);
        }
        if (more) {
          if (!mbar_wait(k_full, ph ^ 1)) { ok = false; break; }
          fence_after_sync();
          if (kb + 1 < nkb_tile[0]) issue_s(0);   // S_A was consumed before p_ready[0] arrived
        }
        if (kb < nkb_tile[1]) {
          if (!mbar_wait(&p_ready[1], ph)) { ok = false; break; }
          fence_after_sync();
          issue_pv(1, kb == 0);
        }
        mma_commit(v_empty);
        if (more) {
          if (kb + 1 < nkb_tile[1]) issue_s(1);
          mma_commit(k_empty);
          if (!mbar_wait(v_empty, ph)) { ok = false; break; }   // both P·V MMAs of this block have read V
          load_v(kb + 1);
        }
      }
      if (!ok) atomicExch(p.status, ATT_ERR_TIMEOUT);
    }
  } else {
    // ---------------------------------------------------------------- softmax / output threads of one tile
    const int g = (warp - 1) >> 2;                   // tile of this warp group
    const int lane_group = warp & 3;                 // TMEM lane quarter this warp may access
    const int row = lane_group * 32 + lane;
    const int qb = qb2 * 2 + g;
    const int t_q = q0 + g * BQ + row;
    const uint32_t lane_addr = uint32_t(lane_group * 32) << 16;
    const uint32_t tmem_s = tmem + g * 128, tmem_pv = tmem + 256 + g * D;
    uint8_t* sPg = sP + g * kPBytes;
    const int my_nkb = nkb_tile[g];
    // m is the reference of the exponentials accumulated so far: p = 2^((s - m) * scale_log2).  It follows the running
    // row maximum lazily — only when the maximum has moved by more than 2^8 past it — so that the output accumulator,
    // which lives in tensor memory and is added to by every P·V product, has to be rescaled on a few blocks only
    // (values of p stay below 2^8, far inside bf16 range; the final division by the row sum uses the same reference).
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int kb = 0; kb < my_nkb; ++kb) {
      if (!mbar_wait(&s_full[g], kb & 1)) { ok = false; break; }
      fence_after_sync();
      const int k0 = kb * BKV;
      const bool need_mask = (p.causal && kb == qb) || (k0 + BKV > p.T);
      // row maximum of this block: two 32-column chunks per TMEM round trip, four independent comparison chains
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 64) {
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(tmem_s + lane_addr + c0, ra);
        tmem_ld_32x32(tmem_s + lane_addr + c0 + 32, rb);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float sa = __uint_as_float(ra[j]), sb = __uint_as_float(rb[j]);
          if (need_mask) {
            const int tk = k0 + c0 + j;
            if (tk >= p.T || (p.causal && tk > t_q)) sa = -INFINITY;
            if (tk + 32 >= p.T || (p.causal && tk + 32 > t_q)) sb = -INFINITY;
          }
          mx4[j & 1] = fmaxf(mx4[j & 1], sa);
          mx4[2 + (j & 1)] = fmaxf(mx4[2 + (j & 1)], sb);
        }
      }
      const float m_blk = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const bool grow = (m_blk - m) * p.scale_log2 > 8.0f;      // true on the first block (m = -inf) of any visible key
      float alpha = 1.0f;
      if (grow) {
        alpha = (m == -INFINITY) ? 0.0f : fast_exp2((m - m_blk) * p.scale_log2);
        m = m_blk;
      }
      const float m_use = (m == -INFINITY) ? 0.0f : m;
      if (kb > 0 && __any_sync(0xffffffffu, grow)) {
        // Some row of this warp moved its reference: scale the accumulated output rows in tensor memory.  The P·V
        // product of the previous block has completed (S of this block was issued after it); the wait makes that
        // ordering explicit and returns at once.
        if (!mbar_wait(&pv_full[g], (kb - 1) & 1)) { ok = false; break; }
        fence_after_sync();
        const float2 a2 = make_float2(alpha, alpha);
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_pv + lane_addr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float2 v = __fmul2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), a2);
            r[j] = __float_as_uint(v.x);
            r[j + 1] = __float_as_uint(v.y);
          }
          tmem_st_32x32(tmem_pv + lane_addr + c0, r);
        }
        tmem_st_wait();
      }
      // p = 2^(s * scale_log2 - m * scale_log2): one packed multiply-add per pair, then the exponential; the row sum
      // is taken over the fp32 values (pairs, packed adds)
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
      const float nm = -m_use * p.scale_log2;
      const float2 nm2 = make_float2(nm, nm);
      float2 rs2 = make_float2(0.0f, 0.0f), rs2b = make_float2(0.0f, 0.0f);
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_s + lane_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          __align__(16) elem2_t hh[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int j = j8 * 8 + 2 * q;
            float2 sv = make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            if (need_mask) {
              const int tk = k0 + c0 + j;
              if (tk >= p.T || (p.causal && tk > t_q)) sv.x = -INFINITY;
              if (tk + 1 >= p.T || (p.causal && tk + 1 > t_q)) sv.y = -INFINITY;
            }
            const float2 e = __ffma2_rn(sv, sc2, nm2);
            const float2 pe = make_float2(fast_exp2(e.x), fast_exp2(e.y));
            if (q & 1) rs2b = __fadd2_rn(rs2b, pe); else rs2 = __fadd2_rn(rs2, pe);
            hh[q] = f22e2(pe);
          }
          const int chunk = (c0 >> 3) + j8;
          uint8_t* dst = sPg + (chunk >> 3) * BQ * 128 + swz(row, chunk & 7);
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(hh);
        }
      }
      l = l * alpha + ((rs2.x + rs2.y) + (rs2b.x + rs2b.y));
      fence_proxy_async();
      fence_before_sync();
      mbar_arrive(&p_ready[g]);
    }
    if (ok && my_nkb > 0) {
      // the last P·V product completes the output rows in tensor memory: divide by the row sum and store
      if (!mbar_wait(&pv_full[g], (my_nkb - 1) & 1)) ok = false;
      fence_after_sync();
      if (ok) {
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        const float2 inv2 = make_float2(inv, inv);
        elem_t* dst = p.out + (((long long)b * p.T + t_q) * p.H + h) * D;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_pv + lane_addr + c0, r);
          tmem_ld_wait();
          if (t_q < p.T) {
#pragma unroll
            for (int d = 0; d < 32; d += 8) {
              __align__(16) elem2_t hh[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                hh[q] = f22e2(__fmul2_rn(
                    make_float2(__uint_as_float(r[d + 2 * q]), __uint_as_float(r[d + 2 * q + 1])), inv2));
              *reinterpret_cast<uint4*>(dst + c0 + d) = *reinterpret_cast<uint4*>(hh);
            }
          }
        }
        if (t_q < p.T && p.lse != nullptr)
          p.lse[((long long)b * p.H + h) * p.T + t_q] = (l > 0.0f) ? m * p.scale + logf(l) : -INFINITY;
      }
      fence_before_sync();
    }
    if (!ok && lane == 0) atomicExch(p.status, ATT_ERR_TIMEOUT);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc(tmem, kTmemCols); }
}

// -------------------------------------------------------------------------------------------------
// backward pre-pass: delta[b,h,t] = sum_d dO*O
// -------------------------------------------------------------------------------------------------
__global__ void attn_delta_kernel(const elem_t* __restrict__ o, const elem_t* __restrict__ d_o, float* __restrict__ delta,
                                  int B, int T, int H, int D, long long do_sb, long long do_st, long long do_sh) {
  const long long idx = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // (b, t, h) row
  const int lane = threadIdx.x & 31;
  if (idx >= (long long)B * T * H) return;
  const int hh = (int)(idx % H);
  const long long bt = idx / H;
  const int t = (int)(bt % T);
  const int b = (int)(bt / T);
  const elem_t* orow = o + idx * D;
  const elem_t* drow = d_o + b * do_sb + t * do_st + hh * do_sh;
  float s = 0.0f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = e22ff(*reinterpret_cast<const elem2_t*>(orow + d));
    const float2 g = e22ff(*reinterpret_cast<const elem2_t*>(drow + d));
    s += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[((long long)b * H + hh) * T + t] = s;
}

// -------------------------------------------------------------------------------------------------
// backward main kernel
// -------------------------------------------------------------------------------------------------
struct AttnBwdParams {
  int B, T, H, D;
  int causal;
  float scale_log2, scale;
  const float* lse;    // (B, H, T)
  const float* delta;  // (B, H, T)
  float* dq;           // (B, T, H, D) fp32, zero-initialised; atomically accumulated
  elem_t* dk;            // (B, T, H, D) contiguous
  elem_t* dv;
  int* status;
};

template <int D>
__global__ void __launch_bounds__(160, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const AttnBwdParams p) {
  constexpr int DP = D / 64;
  constexpr int kTile = 128 * D * 2;           // a 128-row x D operand tile
  constexpr int kSq = 128 * 128 * 2;           // P / dS tiles
  // TMEM columns: S [0,128) — reused for dQ after S has been read; dP [128,256); dV [256,256+D); dK [256+D, 256+2D)
  constexpr uint32_t kTmemCols = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTile;
  uint8_t* sQ = sV + kTile;
  uint8_t* sDO = sQ + kTile;
  uint8_t* sP = sDO + kTile;
  uint8_t* sDS = sP + kSq;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + kSq);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* sdp_full = bars + 2;    // S and dP are in TMEM
  uint64_t* pds_ready = bars + 3;   // P and dS are in smem (128 arrivals)
  uint64_t* dq_full = bars + 4;     // dV/dK accumulated, dQ block in TMEM
  uint64_t* dq_read = bars + 5;     // 128 arrivals: dQ consumed, operands may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k0 = kb * BKV;
  const int nqb = (p.T + BQ - 1) / BQ;
  const int qb_begin = p.causal ? kb : 0;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); prefetch_tensormap(&map_do);
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 128); mbar_init(dq_full, 1); mbar_init(dq_read, 128);
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tm_s = tmem, tm_dp = tmem + 128, tm_dv = tmem + 256, tm_dk = tmem + 256 + D, tm_dq = tmem;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      mbar_expect_tx(kv_full, 2 * kTile);
#pragma unroll
      for (int j = 0; j < DP; ++j) {
        tma_load_attn(sK + j * 128 * 128, &map_k, kv_full, j * 64, h, k0, b);
        tma_load_attn(sV + j * 128 * 128, &map_v, kv_full, j * 64, h, k0, b);
      }
      const uint32_t id_s = make_idesc_f16kind(128, 128, false, false);   // S = Q Kᵀ, dP = dO Vᵀ
      const uint32_t id_t = make_idesc_f16kind(128, D, true, true);       // dV = Pᵀ dO, dK = dSᵀ Q (A, B MN-major)
      const uint32_t id_q = make_idesc_f16kind(128, D, false, true);      // dQ = dS K (B MN-major)
      ok = mbar_wait(kv_full, 0);
      int it = 0;
      for (int qb = qb_begin; qb < nqb && ok; ++qb, ++it) {
        if (it > 0 && !mbar_wait(dq_read, (it - 1) & 1)) { ok = false; break; }   // previous block fully consumed
        mbar_expect_tx(qdo_full, 2 * kTile);
#pragma unroll
        for (int j = 0; j < DP; ++j) {
          tma_load_attn(sQ + j * 128 * 128, &map_q, qdo_full, j * 64, h, qb * BQ, b);
          tma_load_attn(sDO + j * 128 * 128, &map_do, qdo_full, j * 64, h, qb * BQ, b);
        }
        if (!mbar_wait(qdo_full, it & 1)) { ok = false; break; }
        fence_after_sync();
        const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aDO = smem_u32(sDO);
        const uint32_t aP = smem_u32(sP), aDS = smem_u32(sDS);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * 128 * 128 + (k % 4) * 32;
          mma_f16_ss(tm_s, make_smem_desc_sw128(aQ + off, 16, 1024), make_smem_desc_sw128(aK + off, 16, 1024), id_s,
                     k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * 128 * 128 + (k % 4) * 32;
          mma_f16_ss(tm_dp, make_smem_desc_sw128(aDO + off, 16, 1024), make_smem_desc_sw128(aV + off, 16, 1024), id_s,
                     k != 0);
        }
        mma_commit(sdp_full);
        if (!mbar_wait(pds_ready, it & 1)) { ok = false; break; }
        fence_after_sync();
#pragma unroll
        for (int k = 0; k < 128 / 16; ++k) {   // K dimension = queries: 16 rows of P / dS / dO / Q per step
          // A (P or dS) is [query rows][keys]: as an MN-major operand its M = keys; two 64-key panels, LBO = panel
          const uint64_t a_p = make_smem_desc_sw128(aP + k * 16 * 128, 128 * 128, 1024);
          const uint64_t a_ds = make_smem_desc_sw128(aDS + k * 16 * 128, 128 * 128, 1024);
          const uint64_t b_do = make_smem_desc_sw128(aDO + k * 16 * 128, 128 * 128, 1024);
          const uint64_t b_q = make_smem_desc_sw128(aQ + k * 16 * 128, 128 * 128, 1024);
          mma_f16_ss(tm_dv, a_p, b_do, id_t, (it | k) != 0);
          mma_f16_ss(tm_dk, a_ds, b_q, id_t, (it | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < 128 / 16; ++k) {   // dQ = dS (K-major over keys) · K (MN-major: key rows, D contiguous)
          const uint64_t a_ds = make_smem_desc_sw128(aDS + (k / 4) * 128 * 128 + (k % 4) * 32, 16, 1024);
          const uint64_t b_k = make_smem_desc_sw128(aK + k * 16 * 128, 128 * 128, 1024);
          mma_f16_ss(tm_dq, a_ds, b_k, id_q, k != 0);
        }
        mma_commit(dq_full);
      }
      if (!ok) atomicExch(p.status, ATT_ERR_TIMEOUT);
    }
  } else {
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    const uint32_t lane_addr = uint32_t(lane_group * 32) << 16;
    bool ok = true;
    int it = 0;
    for (int qb = qb_begin; qb < nqb; ++qb, ++it) {
      const int t_q = qb * BQ + row;
      const bool row_ok = t_q < p.T;
      const long long stat_idx = ((long long)b * p.H + h) * p.T + t_q;
      const float lse = row_ok ? p.lse[stat_idx] : 0.0f;
      const float dl = row_ok ? p.delta[stat_idx] : 0.0f;
      if (!mbar_wait(sdp_full, it & 1)) { ok = false; break; }
      fence_after_sync();
      const bool need_mask = (p.causal && qb == kb) || (k0 + BKV > p.T) || !row_ok;
#pragma unroll 1
      for (int c0 = 0; c0 < BKV; c0 += 32) {
        uint32_t rs[32], rd[32];
        tmem_ld_32x32(tm_s + lane_addr + c0, rs);
        tmem_ld_32x32(tm_dp + lane_addr + c0, rd);
        tmem_ld_wait();
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          __align__(16) elem2_t hp[4], hd[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float pe[2], de[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int j = j8 * 8 + 2 * q + e;
              const int tk = k0 + c0 + j;
              float pr = fast_exp2(__uint_as_float(rs[j]) * p.scale_log2 - lse * 1.4426950408889634f);
              if (need_mask && (!row_ok || tk >= p.T || (p.causal && tk > t_q))) pr = 0.0f;
              pe[e] = pr;
              de[e] = pr * (__uint_as_float(rd[j]) - dl) * p.scale;
            }
            hp[q] = ff2e2(pe[0], pe[1]);
            hd[q] = ff2e2(de[0], de[1]);
          }
          const int chunk = (c0 >> 3) + j8;
          const uint32_t off = (chunk >> 3) * 128 * 128 + swz(row, chunk & 7);
          *reinterpret_cast<uint4*>(sP + off) = *reinterpret_cast<uint4*>(hp);
          *reinterpret_cast<uint4*>(sDS + off) = *reinterpret_cast<uint4*>(hd);
        }
      }
      fence_proxy_async();
      fence_before_sync();
      mbar_arrive(pds_ready);
      if (!mbar_wait(dq_full, it & 1)) { ok = false; break; }
      fence_after_sync();
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tm_dq + lane_addr + c0, r);
        tmem_ld_wait();
        if (row_ok) {
          float* dst = p.dq + (((long long)b * p.T + t_q) * p.H + h) * D + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 4)       // 16-byte vector reductions: a quarter of the instructions of scalar adds
            atomicAdd(reinterpret_cast<float4*>(dst + j),
                      make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                  __uint_as_float(r[j + 3])));
        }
      }
      fence_before_sync();
      mbar_arrive(dq_read);
    }
    // dK, dV of this key block
    if (ok && it > 0) {
      const int t_k = k0 + row;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        elem_t* base = which == 0 ? p.dv : p.dk;
        const uint32_t src = which == 0 ? tm_dv : tm_dk;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(src + lane_addr + c0, r);
          tmem_ld_wait();
          if (t_k < p.T) {
            elem_t* dst = base + (((long long)b * p.T + t_k) * p.H + h) * D + c0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              __align__(16) elem2_t hh[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                hh[q] = ff2e2(__uint_as_float(r[j + 2 * q]), __uint_as_float(r[j + 2 * q + 1]));
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<uint4*>(hh);
            }
          }
        }
      }
    } else if (ok && it == 0) {
      // no query block attends to this key block (cannot happen for causal self-attention with T_q = T_k)
    }
    if (!ok && lane == 0) atomicExch(p.status, ATT_ERR_TIMEOUT);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc(tmem, kTmemCols); }
}

// -------------------------------------------------------------------------------------------------
// host
// -------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// (B, T, H, D) view with element strides sb, st, sh (inner stride 1); box = 64 x 1 x 128 x 1.
int encode_bthd(CUtensorMap* map, const void* base, int B, int T, int H, int D, long long sb, long long st,
                long long sh) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return 4;
  {  // the driver entry point needs a context current on this thread (see gemm_tcgen05.h)
    static thread_local int bound = -1;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev != bound) {
      cudaSetDevice(dev);
      bound = dev;
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (sb * 2) % 16 || (st * 2) % 16 || (sh * 2) % 16) return 2;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)st * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, ELEM_TMAP, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3;
}

template <typename K>
int set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : 5;
}

}  // namespace

extern "C" {

// q/k/v: (B, T, H, D) views, strides in elements (batch, time, head); out: contiguous (B, T, H, D); lse: (B, H, T).
int fbam_attn_fwd(const void* q, const void* k, const void* v, long long sb, long long st, long long sh, void* out,
                  float* lse, int B, int T, int H, int D, int causal, float scale, int* status, void* stream) {
  if ((D != 64 && D != 128) || B < 1 || T < 1 || H < 1) return 1;
  CUtensorMap mq, mk, mv;
  int e;
  if ((e = encode_bthd(&mq, q, B, T, H, D, sb, st, sh))) return e;
  if ((e = encode_bthd(&mk, k, B, T, H, D, sb, st, sh))) return e;
  if ((e = encode_bthd(&mv, v, B, T, H, D, sb, st, sh))) return e;
  AttnParams p{B, T, H, D, causal, scale * 1.4426950408889634f, scale, (elem_t*)out, lse, status};
  dim3 grid((T + BQ - 1) / BQ, H, B);
  const int stages = D == 64 ? 1 : 2;
  const int smem = BQ * D * 2 + 2 * stages * BKV * D * 2 + BQ * BKV * 2 + 256 + 1024;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 64) {
    if (set_smem(attn_fwd_kernel<64, 1>, smem)) return 5;
    attn_fwd_kernel<64, 1><<<grid, 160, smem, s>>>(mq, mk, mv, p);
  } else {
    if (set_smem(attn_fwd_kernel<128, 2>, smem)) return 5;
    attn_fwd_kernel<128, 2><<<grid, 160, smem, s>>>(mq, mk, mv, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

// Variant of fbam_attn_fwd with two query tiles per CTA (attn_fwd2_kernel); same arguments and results.
int fbam_attn_fwd2(const void* q, const void* k, const void* v, long long sb, long long st, long long sh, void* out,
                   float* lse, int B, int T, int H, int D, int causal, float scale, int* status, void* stream) {
  if ((D != 64 && D != 128) || B < 1 || T < 1 || H < 1) return 1;
  CUtensorMap mq, mk, mv;
  int e;
  if ((e = encode_bthd(&mq, q, B, T, H, D, sb, st, sh))) return e;
  if ((e = encode_bthd(&mk, k, B, T, H, D, sb, st, sh))) return e;
  if ((e = encode_bthd(&mv, v, B, T, H, D, sb, st, sh))) return e;
  AttnParams p{B, T, H, D, causal, scale * 1.4426950408889634f, scale, (elem_t*)out, lse, status};
  dim3 grid((T + 2 * BQ - 1) / (2 * BQ), H, B);
  const int smem = 2 * BQ * D * 2 + 2 * BKV * D * 2 + 2 * BQ * BKV * 2 + 256 + 1024;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 64) {
    if (set_smem(attn_fwd2_kernel<64>, smem)) return 5;
    attn_fwd2_kernel<64><<<grid, 288, smem, s>>>(mq, mk, mv, p);
  } else {
    if (set_smem(attn_fwd2_kernel<128>, smem)) return 5;
    attn_fwd2_kernel<128><<<grid, 288, smem, s>>>(mq, mk, mv, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

// d_o: (B, T, H, D) view with its own strides; o: contiguous forward output; dq: fp32 zero-initialised (B,T,H,D);
// dk/dv: contiguous bf16 (B,T,H,D); delta: (B,H,T) scratch.
int fbam_attn_bwd(const void* q, const void* k, const void* v, long long sb, long long st, long long sh, const void* o,
                  const void* d_o, long long do_sb, long long do_st, long long do_sh, const float* lse, float* delta,
                  float* dq, void* dk, void* dv, int B, int T, int H, int D, int causal, float scale, int* status,
                  void* stream) {
  if ((D != 64 && D != 128) || B < 1 || T < 1 || H < 1) return 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * T * H;
  attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const elem_t*)o, (const elem_t*)d_o, delta, B, T, H, D,
                                                               do_sb, do_st, do_sh);
  if (cudaGetLastError() != cudaSuccess) return 5;
  CUtensorMap mq, mk, mv, mdo;
  int e;
  if ((e = encode_bthd(&mq, q, B, T, H, D, sb, st, sh))) return e;
  if ((e = encode_bthd(&mk, k, B, T, H, D, sb, st, sh))) return e;
  if ((e = encode_bthd(&mv, v, B, T, H, D, sb, st, sh))) return e;
  if ((e = encode_bthd(&mdo, d_o, B, T, H, D, do_sb, do_st, do_sh))) return e;
  AttnBwdParams p{B, T, H, D, causal, scale * 1.4426950408889634f, scale, lse, delta, dq, (elem_t*)dk, (elem_t*)dv, status};
  dim3 grid((T + BKV - 1) / BKV, H, B);
  const int smem = 4 * 128 * D * 2 + 2 * 128 * 128 * 2 + 256 + 1024;
  if (D == 64) {
    if (set_smem(attn_bwd_kernel<64>, smem)) return 5;
    attn_bwd_kernel<64><<<grid, 160, smem, s>>>(mq, mk, mv, mdo, p);
  } else {
    if (set_smem(attn_bwd_kernel<128>, smem)) return 5;
    attn_bwd_kernel<128><<<grid, 160, smem, s>>>(mq, mk, mv, mdo, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

}  // extern "C"
