// Two-SM ("cta_group::2") variant of the tcgen05 GEMM / implicit-GEMM convolution.
//
// Two CTAs on neighbouring SMs form a cluster and compute one 256 x BN output tile together: each CTA loads its
// own 128 rows of A and HALF of the B tile (BN/2 rows) into its shared memory, and a single thread of the leader
// CTA issues tcgen05.mma.cta_group::2 instructions that run on both SMs' tensor cores — each SM multiplies its own
// A rows with the whole B tile, reading the other half from the peer's shared memory.  Per SM that is 32 KB of
// operands per 512 tensor-core cycles (64 B/clk) instead of 48 KB for a stand-alone 128 x 256 tile, and — unlike
// the single-CTA 256 x 256 tile — each SM still has room for TWO accumulators in tensor memory, so the epilogue of
// tile i overlaps the main loop of tile i+1.
//
// Synchronisation: TMA loads of both CTAs complete on the LEADER's "full" barrier (cp.async.bulk.tensor with
// .cta_group::2 and the barrier address of the leader; no multicast anywhere); tcgen05.commit arrives on both CTAs'
// "empty" / "tmem_full" barriers at once; the epilogue warps of the second CTA release the accumulator by a remote
// arrive on the leader's "tmem_empty" barrier.  All waits are bounded; the cluster is re-joined before exit.
//
// Same operation set as gemm_tcgen05.cu (reference kernel families: cutlass_codegen/gemm_cutlass_kernel.cu:198-330,
// cutlass_codegen/conv2d_cutlass_kernel.cu).
#include "gemm_epilogue.cuh"
#include <cstring>

#include "gemm_tcgen05.h"
#include "gemm_out_maps.h"
#include "tc05.cuh"

extern int g_fbam_reserved_sms;        // defined in gemm_tcgen05.cu
extern int g_fbam_last_driver_error;   // defined in gemm_tcgen05.cu

namespace {

using namespace tc05;

constexpr int BM = 128;   // rows per CTA (256 per pair)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (2 + kEpiWarps);

template <int BN>
struct Smem2 {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = (BN / 2) * BK * 2;   // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  static constexpr int kEpiStage = kEpiWarps * 2 * 2048;   // per epilogue warp: two 32-row x 64-byte buffers for TMA stores
  static constexpr int kTotal = kStages * kStageBytes + kEpiStage + 512 + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA loads whose completion is counted on the barrier at `bar_cluster_addr` (the leader's copy).
__device__ __forceinline__ void tma2_load_2d(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma2_load_4d(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                             int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
      "%6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma2_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at the same shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void mma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

// Row of this CTA's 128-row half -> element offset in D (or -1).  `half_tile` indexes 128-row tiles / bricks.
__device__ __forceinline__ long long row_offset2(const GemmParams& p, int half_tile, int row, int off_h, int off_w) {
  if (p.mode != GEMM_MODE_CONV) {
    const int m = half_tile * BM + row;
    return m < p.M ? (long long)m * p.ldd : -1;
  }
  const ConvGeom& g = p.conv;
  const int wb = half_tile % g.tiles_w;
  const int hb = (half_tile / g.tiles_w) % g.tiles_h;
  const int nb = half_tile / (g.tiles_w * g.tiles_h);
  const int wl = row % g.tw, hl = (row / g.tw) % g.th, nl = row / (g.tw * g.th);
  const int n = nb * g.tn + nl, h = hb * g.th + hl, w = wb * g.tw + wl;
  if (n >= g.batch || h >= g.grid_h || w >= g.grid_w) return -1;
  const int oh = h * g.out_mul + off_h, ow = w * g.out_mul + off_w;
  if (oh >= g.out_h || ow >= g.out_w) return -1;
  return (((long long)n * g.out_h + oh) * g.out_w + ow) * p.ldd;
}

// Work items of one CTA pair: tile `cluster_id + j * num_clusters` for j = 0, 1, ..., each visited once per parity
// class (all classes of a tile back to back).  The three roles walk the same sequence.
struct WorkIter {
  int tile, cls;
  __device__ __forceinline__ WorkIter(int first) : tile(first), cls(0) {}
  __device__ __forceinline__ void next(int ncls, int stride) {
    if (++cls >= ncls) { cls = 0; tile += stride; }
  }
};

// p.tiles_m counts PAIR tiles (256 rows); K is never split in this variant.
template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_pre, const GemmParams p) {
  using L = Smem2<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + L::kStages * L::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + L::kEpiStage);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* tmem_full = empty_bar + L::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int cluster_id = blockIdx.x / 2, num_clusters = gridDim.x / 2;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = p.tiles_m * tiles_n;
  const int ncls = p.num_classes > 0 ? p.num_classes : 1;
  constexpr uint32_t kTmemCols = 2 * BN;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    if (p.tma_store >= 1) prefetch_tensormap(&map_d);
    if (p.tma_store >= 2) prefetch_tensormap(&map_pre);
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);    // leader: one arrive.expect_tx covering both CTAs' bytes
      mbar_init(&empty_bar[s], 1);   // one multicast commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 2 * kEpiWarps);   // leader: epilogue warps of both CTAs
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, kTmemCols);
    tmem_relinquish2();
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before anyone signals across the pair
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (WorkIter it(cluster_id); it.tile < num_tiles && ok; it.next(ncls, num_clusters)) {
        const int tile = it.tile;
        const int tile_m = (tile / tiles_n + p.tile_m_rotate) % p.tiles_m, tile_n = tile % tiles_n;
        const int half = tile_m * 2 + (int)rank;              // this CTA's 128-row tile / brick
        const int b_row0 = tile_n * BN + (int)rank * (BN / 2);   // this CTA's half of the B tile
        const bool classes = p.num_classes > 0;
        const int k_blocks = classes ? p.cls[it.cls].num_taps * p.conv.c_blocks : p.k_blocks;
        const int kb_base = classes ? p.cls[it.cls].k_block_base : 0;
        int cn = 0, ch = 0, cw = 0;
        if (p.mode == GEMM_MODE_CONV) {
          const ConvGeom& g = p.conv;
          cw = (half % g.tiles_w) * g.tw * g.in_mul;
          ch = ((half / g.tiles_w) % g.tiles_h) * g.th * g.in_mul;
          cn = (half / (g.tiles_w * g.tiles_h)) * g.tn;
        }
        if (p.ready_flags != nullptr) {
          // all-gather -> GEMM: wait (bounded) until the peers' shards that this CTA's loads read have landed
          const int r0 = p.flag_on_b ? b_row0 : half * BM;
          const int r1 = min(p.flag_on_b ? p.N : p.M, r0 + (p.flag_on_b ? BN / 2 : BM)) - 1;
          for (int f = r0 / p.flag_rows; f <= r1 / p.flag_rows && ok; ++f) {
            unsigned spins = 0, v;
            do {
              asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.ready_flags + f) : "memory");
              if ((int)(v - p.flag_epoch) >= 0) break;
              __nanosleep(64);
            } while (++spins < p.flag_spin_limit);
            if ((int)(v - p.flag_epoch) < 0) ok = false;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy acquire -> async-proxy (TMA) reads
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          if (p.mode == GEMM_MODE_CONV) {
            const ConvGeom& g = p.conv;
            const int tap = kb / g.c_blocks, cb = kb % g.c_blocks;
            const int dw = classes ? p.cls[it.cls].tap_dw[tap] : g.tap_dw[tap];
            const int dh = classes ? p.cls[it.cls].tap_dh[tap] : g.tap_dh[tap];
            tma2_load_4d(sa, &map_a, leader_full, cb * BK, cw + dw, ch + dh, cn);
          } else if (p.a_mn_major) {
            tma2_load_2d(sa, &map_a, leader_full, half * BM, kb * BK);
            tma2_load_2d(sa + BK * 128, &map_a, leader_full, half * BM + 64, kb * BK);
          } else {
            tma2_load_2d(sa, &map_a, leader_full, kb * BK, half * BM);
          }
          if (p.b_mn_major) {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              tma2_load_2d(sb + j * BK * 128, &map_b, leader_full, b_row0 + j * 64, (kb_base + kb) * BK);
          } else {
            tma2_load_2d(sb, &map_b, leader_full, (kb_base + kb) * BK, b_row0);
          }
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) atomicExch(p.status, GEMM_ERR_PRODUCER_TIMEOUT);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc_f16kind(256, BN, p.a_mn_major != 0, p.b_mn_major != 0);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (WorkIter it(cluster_id); it.tile < num_tiles && ok; it.next(ncls, num_clusters)) {
        const int k_blocks = p.num_classes > 0 ? p.cls[it.cls].num_taps * p.conv.c_blocks : p.k_blocks;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
          fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            mma2_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          mma2_commit_both(&empty_bar[stage]);
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma2_commit_both(&tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) atomicExch(p.status, GEMM_ERR_MMA_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs, own rows)
    const int lane_group = warp % 4;
    const int col_half = (warp - 2) / 4;
    const int row = lane_group * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0, stage_turn = 0;
    bool ok = true;
    for (WorkIter it(cluster_id); it.tile < num_tiles && ok; it.next(ncls, num_clusters)) {
      const int tile = it.tile;
      const int tile_m = (tile / tiles_n + p.tile_m_rotate) % p.tiles_m, tile_n = tile % tiles_n;
      const int half = tile_m * 2 + (int)rank;
      const int off_h = p.num_classes > 0 ? p.cls[it.cls].out_off_h : p.conv.out_off_h;
      const int off_w = p.num_classes > 0 ? p.cls[it.cls].out_off_w : p.conv.out_off_w;
      const long long roff = row_offset2(p, half, row, off_h, off_w);
      // TMA stores: where in the output this warp's 32 rows start (a box of st_bn x st_bh x st_bw output positions of
      // the brick for a convolution, 32 matrix rows otherwise); a box that starts outside the output is skipped,
      // one that reaches over its edge is clipped by the copy.
      int sx1 = 0, sx2 = 0, sx3 = 0;
      bool box_in = true;
      if (p.tma_store) {
        if (p.mode == GEMM_MODE_CONV) {
          const ConvGeom& g = p.conv;
          const int r0 = lane_group * 32;
          const int w = (half % g.tiles_w) * g.tw + r0 % g.tw;
          const int h = ((half / g.tiles_w) % g.tiles_h) * g.th + (r0 / g.tw) % g.th;
          const int n = (half / (g.tiles_w * g.tiles_h)) * g.tn + r0 / (g.tw * g.th);
          sx1 = w * g.out_mul + off_w;
          sx2 = h * g.out_mul + off_h;
          sx3 = n;
          box_in = n < g.batch && h < g.grid_h && w < g.grid_w && sx1 < g.out_w && sx2 < g.out_h;
        } else {
          sx1 = half * BM + lane_group * 32;
          box_in = sx1 < p.M;
        }
      }
      uint8_t* stage_pre = epi_stage + (warp - 2) * 4096;
      uint8_t* stage_out = stage_pre + 2048;
      // the side input (gelu_grad_in or residual) of the first chunk is requested before the accumulator is waited
      // for, and that of every later chunk before the previous one is processed
      const int c_first = col_half * (BN / 2), c_last = (col_half + 1) * (BN / 2);
      const elem_t* aux_row = gemm_epi::aux_row_ptr(p, roff);
      uint4 aux[4] = {};
      gemm_epi::aux_prefetch(aux_row, tile_n * BN + c_first, p.N, aux);
      if (!mbar_wait(&tmem_full[acc], acc_phase)) { ok = false; break; }
      fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(lane_group * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c0 = c_first; c0 < c_last; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        const int n0 = tile_n * BN + c0;
        uint4 cur[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) cur[q] = aux[q];
        if (c0 + 32 < c_last) gemm_epi::aux_prefetch(aux_row, n0 + 32, p.N, aux);
        tmem_ld_wait();
        if (n0 >= p.N) continue;                               // the same for the whole warp
        if (p.tma_store && n0 + 32 <= p.N) {
          // A staging buffer is free once the copy that read it is done (tracked by lane 0, which issued it).  Without
          // preact_out the two buffers take turns (stage_turn counts this warp's stored chunks across tiles), so only
          // the copy before the previous one has to be done.
          const bool both = p.tma_store >= 2;
          uint8_t* out_buf = (both || (stage_turn++ & 1)) ? stage_out : stage_pre;
          if (lane == 0) {
            if (both) bulk_wait_group_read<0>();
            else bulk_wait_group_read<1>();
          }
          __syncwarp();
          gemm_epi::store_chunk<false, true, true>(p, roff, n0, r, cur, stage_pre, out_buf);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (box_in) {
              if (p.mode == GEMM_MODE_CONV) {
                if (both) tma_store_4d(&map_pre, stage_pre, n0, sx1, sx2, sx3);
                tma_store_4d(&map_d, out_buf, n0, sx1, sx2, sx3);
              } else {
                if (both) tma_store_2d(&map_pre, stage_pre, n0, sx1);
                tma_store_2d(&map_d, out_buf, n0, sx1);
              }
            }
            bulk_commit_group();      // also when nothing was stored: the group count paces the buffers
          }
          continue;
        }
        if (roff < 0) continue;
        gemm_epi::store_chunk<false, true>(p, roff, n0, r, cur);
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&tmem_empty[acc]);
        else remote_arrive(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0) atomicExch(p.status, GEMM_ERR_EPILOGUE_TIMEOUT);
    if (lane == 0) bulk_wait_group_all();     // this warp's TMA stores have left shared memory and reached global memory
  }

  fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves (and frees shared / tensor memory) while the other may still touch it
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn2() {
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
int enc2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn enc = encode_fn2();
  if (!enc) return GEMM_ERR_DRIVER;
  fbam_bind_context_to_thread();
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return GEMM_ERR_ALIGNMENT;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, ELEM_TMAP, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_fbam_last_driver_error = (int)r;
  return r == CUDA_SUCCESS ? 0 : GEMM_ERR_TENSORMAP;
}
int enc_nhwc(CUtensorMap* map, const void* base, int n, int h, int w, int c, int tn, int th, int tw, int stride) {
  EncodeTiledFn enc = encode_fn2();
  if (!enc) return GEMM_ERR_DRIVER;
  fbam_bind_context_to_thread();
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (c * 2) % 16) return GEMM_ERR_ALIGNMENT;
  cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)c * 2, (cuuint64_t)w * c * 2, (cuuint64_t)h * w * c * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)((tw - 1) * stride + 1), (cuuint32_t)((th - 1) * stride + 1), (cuuint32_t)tn};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  return enc(map, ELEM_TMAP, 4, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : GEMM_ERR_TENSORMAP;
}

template <int BN>
int launch2(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
  using L = Smem2<BN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm2_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
      return GEMM_ERR_LAUNCH;
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = p.tiles_m * ((p.N + BN - 1) / BN);
  const int usable = sms - g_fbam_reserved_sms > 2 ? sms - g_fbam_reserved_sms : 2;
  int clusters = tiles < usable / 2 ? tiles : usable / 2;
  if (p.max_ctas > 1 && clusters > p.max_ctas / 2) clusters = p.max_ctas / 2;
  CUtensorMap md, mpre;
  const int e = fbam_encode_out_maps(encode_fn2(), &md, &mpre, p);
  if (e) return e;
  gemm2_kernel<BN><<<2 * clusters, kThreads, L::kTotal, stream>>>(ma, mb, md, mpre, p);
  return cudaGetLastError() == cudaSuccess ? 0 : GEMM_ERR_LAUNCH;
}

}  // namespace

// Same contracts as fbam_gemm / fbam_conv (gemm_tcgen05.cu), computed by CTA pairs.  N must be a
// multiple of 16 with BN in {128, 256}; split-K stays on the single-CTA kernel.
extern "C" int fbam_gemm2(const void* A, long long lda, int a_mn_major, const void* B, long long ldb,
                               int b_mn_major, int M, int N, int K, GemmParams* params, void* stream) {
  GemmParams p = *params;
  if (M <= 0 || N <= 0 || K <= 0 || p.splits > 1) return GEMM_ERR_SHAPE;
  if (p.ready_flags != nullptr && p.flag_rows <= 0) return GEMM_ERR_SHAPE;
  if (p.flag_spin_limit == 0) p.flag_spin_limit = 1u << 22;
  p.mode = GEMM_MODE_PLAIN;
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.k_blocks = (K + BK - 1) / BK;
  p.splits = 1;
  const int bn = (p.bn == 128 || N <= 128) ? 128 : 256;
  p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int elt = p.out_fp32 ? 4 : 2;
  p.vec_ok = (p.ldd % (16 / elt) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
             (p.preact_out == nullptr || (reinterpret_cast<uintptr_t>(p.preact_out) & 15) == 0) &&
             (p.gelu_grad_in == nullptr || (reinterpret_cast<uintptr_t>(p.gelu_grad_in) & 15) == 0) &&
             (p.residual == nullptr || (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0) && (p.ldd % 8 == 0);
  if (p.rs_rows_per_rank > 0) p.vec_ok = (p.ldd % (p.rs_slot_plus1 > 0 ? 8 : 4) == 0);
  CUtensorMap ma, mb;
  int e = a_mn_major ? enc2d(&ma, A, K, M, lda, 64) : enc2d(&ma, A, M, K, lda, BM);
  if (e) return e;
  e = b_mn_major ? enc2d(&mb, B, K, N, ldb, 64) : enc2d(&mb, B, N, K, ldb, bn / 2);
  if (e) return e;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return bn == 128 ? launch2<128>(ma, mb, p, s) : launch2<256>(ma, mb, p, s);
}

extern "C" int fbam_conv2(const void* X, int in_h, int in_w, int C, const void* Wmat, long long ldw, int N,
                               GemmParams* params, void* stream) {
  GemmParams p = *params;
  ConvGeom& g = p.conv;
  if (C % 64 != 0 || g.tn * g.th * g.tw != BM || g.num_taps < 1 || g.num_taps > 9) return GEMM_ERR_SHAPE;
  if (p.num_classes < 0 || p.num_classes > 4) return GEMM_ERR_SHAPE;
  int class_taps = 0;
  for (int c = 0; c < p.num_classes; ++c) {
    if (p.cls[c].num_taps < 1 || p.cls[c].num_taps > 4 || p.cls[c].k_block_base != class_taps * (C / 64)) return GEMM_ERR_SHAPE;
    class_taps += p.cls[c].num_taps;
  }
  if (p.num_classes > 0 && class_taps != g.num_taps) return GEMM_ERR_SHAPE;   // conv.num_taps = all classes' taps
  p.mode = GEMM_MODE_CONV;
  p.a_mn_major = 0; p.b_mn_major = 0;
  g.c_blocks = C / 64;
  g.tiles_w = (g.grid_w + g.tw - 1) / g.tw;
  g.tiles_h = (g.grid_h + g.th - 1) / g.th;
  const int half_tiles = g.tiles_w * g.tiles_h * ((g.batch + g.tn - 1) / g.tn);
  p.tiles_m = (half_tiles + 1) / 2;
  p.M = half_tiles * BM;
  p.N = N; p.K = g.num_taps * C;
  p.k_blocks = g.num_taps * g.c_blocks;
  p.splits = 1;
  const int bn = (p.bn == 128 || N <= 128) ? 128 : 256;
  const int elt = p.out_fp32 ? 4 : 2;
  p.vec_ok = (p.ldd % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) && (p.ldd % (16 / elt) == 0);
  CUtensorMap ma, mb;
  int e = enc_nhwc(&ma, X, g.batch, in_h, in_w, C, g.tn, g.th, g.tw, g.in_mul);
  if (e) return e;
  e = enc2d(&mb, Wmat, N, p.K, ldw, bn / 2);
  if (e) return e;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return bn == 128 ? launch2<128>(ma, mb, p, s) : launch2<256>(ma, mb, p, s);
}
