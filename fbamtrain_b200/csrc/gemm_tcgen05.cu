// Persistent, warp-specialised bf16 GEMM / implicit-GEMM convolution for sm_100a.
//
//   D[M, N] = epilogue( A[M, K] · B[N, K]ᵀ )        fp32 accumulation in tensor memory
//
// One CTA per SM loops over 128 x BN output tiles.  Warp 0 streams operand tiles into a 4-stage
// shared-memory ring with TMA (128-byte swizzle); warp 1 issues tcgen05.mma (one elected thread)
// into one of two TMEM accumulators; warps 2-5 drain the other accumulator with tcgen05.ld, apply the
// fused epilogue and store — so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Operand sources (template MODE):
//   GEMM   A and B are 2-D matrices.  Each may be K-major (row = M/N index, K contiguous) or MN-major
//          (row = K index, M/N contiguous); MN-major tiles are fetched as 64-wide column panels and
//          consumed through the transposed-operand form of the UMMA descriptor, so weight-gradient
//          products (Xᵀ·dY) need no explicit transposes.
//   CONV   A is an NHWC activation tensor reached through a 4-D tensor map; a K block is one filter
//          tap x 64 input channels, and the tile's 128 rows are a TN x TH x TW brick of output pixels,
//          so the im2col gather is done by TMA (element strides give the convolution stride, out-of-
//          range coordinates give zero padding).  Forward and data-gradient convolutions both map
//          onto this mode (the data gradient of a stride-2 convolution is four parity classes, each a
//          stride-1 gather over the taps that reach that parity).
//
// Epilogue (runtime flags): + bias[n], GELU (optionally storing the pre-activation), + residual[m, n],
// x gelu'(aux[m, n]) (fuses the activation gradient into the GEMM that produces dH), C += (fp32
// accumulate-into-output), bf16 or fp32 output.
//
// Every mbarrier wait is bounded; on timeout the CTA writes an error code to `status` and unwinds.
//
// Takes the place of the reference's GEMM and convolution kernel families: matmul / addmm / addmm_gelu[_preact] /
// matmul_gelu_bwd with transposed-operand, fp32-output and accumulate variants (reference:
// kernel_gen/kernel_gen/kernels/cutlass_codegen/gemm_cutlass_kernel.cu:198-330, kernels/matmul.py), the fusions
// its matmul pass selects (src/passes/matmul_pass.cpp:2783-3468), and conv2d fprop / dgrad / wgrad with
// accumulation (cutlass_codegen/conv2d_cutlass_kernel.cu, kernels/conv2d.py:72-190, kernels/conv2d_bwd.py:6-232;
// dispatch in src/passes/conv2d_pass.cpp).
#include "gemm_tcgen05.h"
#include "gemm_out_maps.h"
#include <cstddef>
#include "gemm_epilogue.cuh"
#include "tc05.cuh"

// SMs the persistent kernels leave free (see fbam_set_reserved_sms).
int g_fbam_reserved_sms = 0;
// Result code of the last failed tensor-map encode (diagnostics: fbam_last_driver_error).
int g_fbam_last_driver_error = 0;

namespace {

using namespace tc05;

constexpr int BK = 64;       // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kNumEpilogueWarps = 8;   // two warps per TMEM lane group, each draining half of the columns
constexpr int kThreads = 32 * (2 + kNumEpilogueWarps);

// BM = 128: two TMEM accumulators of BN columns alternate between tiles (epilogue overlaps the next main loop).
// BM = 256: the tile is two stacked M = 128 halves that share every B fetch — 64 B of operand traffic per
//           tensor-core cycle instead of 96 — at the price of using both accumulators for one tile.
template <int BM, int BN>
struct SmemLayout {
  static constexpr int kStageRaw = (BM + BN) * BK * 2;
  static constexpr int kStages = (200 * 1024 / kStageRaw) > 6 ? 6 : (200 * 1024 / kStageRaw);
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kEpiStage = 8 * 2 * 2048;   // per epilogue warp: two 32-row x 64-byte buffers for TMA stores
  static constexpr int kTotal = kStages * kStageBytes + kEpiStage + kBarrierBytes + 1024;  // +1024: manual alignment slack
};

// Row of the output tile -> element offset of that row in D (or -1 when the row is out of range).
__device__ __forceinline__ long long row_offset(const GemmParams& p, int tile_m, int row, int BM) {
  if (p.mode != GEMM_MODE_CONV) {
    int m = tile_m * BM + row;
    return m < p.M ? (long long)m * p.ldd : -1;
  }
  // CONV: tile_m enumerates (n-brick, h-brick, w-brick)
  const ConvGeom& g = p.conv;
  int wb = tile_m % g.tiles_w;
  int hb = (tile_m / g.tiles_w) % g.tiles_h;
  int nb = tile_m / (g.tiles_w * g.tiles_h);
  int wl = row % g.tw, hl = (row / g.tw) % g.th, nl = row / (g.tw * g.th);
  int n = nb * g.tn + nl, h = hb * g.th + hl, w = wb * g.tw + wl;
  if (n >= g.batch || h >= g.grid_h || w >= g.grid_w) return -1;
  int oh = h * g.out_mul + g.out_off_h, ow = w * g.out_mul + g.out_off_w;
  if (oh >= g.out_h || ow >= g.out_w) return -1;
  return (((long long)n * g.out_h + oh) * g.out_w + ow) * p.ldd;
}

// Work item = (split, tile_m, tile_n): output tile plus the range of K blocks this CTA accumulates.
// With split-K, split s takes K blocks s, s + splits, s + 2*splits, ...: concurrently running CTAs then stream
// through neighbouring addresses together instead of starting many far-apart streams whose strides can all fall
// onto the same memory channels.
struct Work {
  int tile_m, tile_n, k_begin, k_end, k_step, split;
};
__device__ __forceinline__ Work decode_work(const GemmParams& p, int item, int tiles_n) {
  Work w;
  const int tiles = p.tiles_m * tiles_n;
  const int split = item / tiles;
  const int t = item % tiles;
  w.split = split;
  w.tile_m = t / tiles_n;
  w.tile_n = t % tiles_n;
  if (p.tile_m_rotate > 0) w.tile_m = (w.tile_m + p.tile_m_rotate) % p.tiles_m;
  w.k_begin = split;
  w.k_end = p.k_blocks;
  w.k_step = p.splits;
  return w;
}

// CE: the instantiation that carries the fused LM-head + cross-entropy epilogues (GemmParams::ce_mode); the plain
// instantiations are compiled without them, so their register use does not change.
template <int BM, int BN, bool CE = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_pre, const GemmParams p) {
  using L = SmemLayout<BM, BN>;
  constexpr int MH = BM / 128;  // M = 128 halves per tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + L::kStages * L::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_stage + L::kEpiStage);
  uint64_t* empty_bar = full_bar + L::kStages;
  uint64_t* tmem_full = empty_bar + L::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = p.tiles_m * tiles_n * p.splits;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    if (p.tma_store >= 1) prefetch_tensormap(&map_d);
    if (p.tma_store >= 2) prefetch_tensormap(&map_pre);
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], kNumEpilogueWarps);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Work wk = decode_work(p, tile, tiles_n);
        const int tile_m = wk.tile_m, tile_n = wk.tile_n;
        int cn = 0, ch = 0, cw = 0;
        if (p.mode == GEMM_MODE_CONV) {
          const ConvGeom& g = p.conv;
          cw = (tile_m % g.tiles_w) * g.tw * g.in_mul;
          ch = ((tile_m / g.tiles_w) % g.tiles_h) * g.th * g.in_mul;
          cn = (tile_m / (g.tiles_w * g.tiles_h)) * g.tn;
        }
        if (p.ready_flags != nullptr) {
          // all-gather -> GEMM: wait (bounded) until the peers' shards that this tile reads have landed
          const int r0 = p.flag_on_b ? tile_n * BN : tile_m * BM;
          const int r1 = min(p.flag_on_b ? p.N : p.M, r0 + (p.flag_on_b ? BN : BM)) - 1;
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
        for (int kb = wk.k_begin; kb < wk.k_end; kb += wk.k_step) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          if (p.mode == GEMM_MODE_WGRAD) {
            // K block = brick of 64 output pixels; A = dY panel pair, B = gathered input for this tile's tap
            const ConvGeom& g = p.conv;
            const int bw = (kb % g.tiles_w) * g.tw;
            const int bh = ((kb / g.tiles_w) % g.tiles_h) * g.th;
            const int bn = (kb / (g.tiles_w * g.tiles_h)) * g.tn;
            const int C = g.c_blocks * 64;
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_4d(sa + j * BK * 128, &map_a, &full_bar[stage], tile_m * BM + j * 64, bw, bh, bn);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              // column panel j of the tile: its filter tap and channel offset (past the last tap: channel
              // coordinate C, i.e. out of range, which TMA fills with zeros)
              const int col = tile_n * BN + j * 64;
              int tap = col / C, c0 = col % C;
              if (tap >= g.num_taps) { tap = 0; c0 = C; }
              tma_load_4d(sb + j * BK * 128, &map_b, &full_bar[stage], c0, bw * g.in_mul + g.tap_dw[tap],
                          bh * g.in_mul + g.tap_dh[tap], bn);
            }
            if (++stage == L::kStages) { stage = 0; phase ^= 1; }
            continue;
          }
          if (p.mode == GEMM_MODE_CONV) {
            const ConvGeom& g = p.conv;
            const int tap = kb / g.c_blocks, cb = kb % g.c_blocks;
            tma_load_4d(sa, &map_a, &full_bar[stage], cb * BK, cw + g.tap_dw[tap], ch + g.tap_dh[tap], cn);
          } else if (p.a_mn_major) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * BK * 128, &map_a, &full_bar[stage], tile_m * BM + j * 64, kb * BK);
          } else {
            tma_load_2d(sa, &map_a, &full_bar[stage], kb * BK, tile_m * BM);
          }
          if (p.b_mn_major) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * BK * 128, &map_b, &full_bar[stage], tile_n * BN + j * 64, kb * BK);
          } else {
            tma_load_2d(sb, &map_b, &full_bar[stage], kb * BK, tile_n * BN);
          }
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) atomicExch(p.status, GEMM_ERR_PRODUCER_TIMEOUT);
      // (a timed-out flag wait also lands here: the consumers then time out on their barriers and the CTA unwinds)
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_f16kind(128, BN, p.a_mn_major != 0, p.b_mn_major != 0);
      // K-major: 8-row groups are 1024 B apart (SBO); one UMMA_K step = 32 B inside the swizzle row.
      // MN-major: 64-wide column panels are BK*128 B apart (LBO), 8-row K groups 1024 B apart (SBO);
      //           one UMMA_K step = 16 rows = 2048 B.
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Work wk = decode_work(p, tile, tiles_n);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (MH == 1 ? acc * BN : 0);
        for (int kb = wk.k_begin; kb < wk.k_end; kb += wk.k_step) {
          if (!mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
          fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t db = make_smem_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
#pragma unroll
            for (int h = 0; h < MH; ++h) {   // M half h: rows [128h, 128h+128) = 16 KB further in either layout
              const uint64_t da = make_smem_desc_sw128(sa + h * 128 * 128 + k * a_kstep, a_lbo, 1024);
              mma_f16_ss(d_tmem + h * BN, da, db, idesc, ((kb - wk.k_begin) | k) != 0);   // first block overwrites
            }
          }
          mma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == L::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&tmem_full[acc]);
        if (MH == 2) { acc_phase ^= 1; }
        else if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) atomicExch(p.status, GEMM_ERR_MMA_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int lane_group = warp % 4;  // TMEM lanes [32*lane_group, +32) are visible to this warp
    const int second = (warp - 2) / 4;  // BM=128: second half of the columns; BM=256: second M half
    const int row = (MH == 2 ? second * 128 : 0) + lane_group * 32 + lane;
    const int c_begin = MH == 2 ? 0 : second * (BN / 2), c_end = MH == 2 ? BN : (second + 1) * (BN / 2);
    int acc = 0;
    uint32_t acc_phase = 0, stage_turn = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const Work wk = decode_work(p, tile, tiles_n);
      const int tile_m = wk.tile_m, tile_n = wk.tile_n;
      // the side input of the first chunk is requested before the accumulator is waited for, and that of every
      // later chunk before the previous one is processed
      const long long roff = row_offset(p, tile_m, row, BM);
      const elem_t* aux_row = gemm_epi::aux_row_ptr(p, roff);
      uint4 aux[4] = {};
      gemm_epi::aux_prefetch(aux_row, tile_n * BN + c_begin, p.N, aux);
      // TMA stores: where in the output this warp's 32 rows start (a box of st_bn x st_bh x st_bw output positions of
      // the brick for a convolution, 32 matrix rows otherwise); a box that starts outside the output is skipped,
      // one that reaches over its edge is clipped by the copy.
      int sx1 = 0, sx2 = 0, sx3 = 0;
      bool box_in = true;
      if (!CE && p.tma_store) {
        const int r0 = (MH == 2 ? second * 128 : 0) + lane_group * 32;
        if (p.mode == GEMM_MODE_CONV) {
          const ConvGeom& g = p.conv;
          const int w = (tile_m % g.tiles_w) * g.tw + r0 % g.tw;
          const int h = ((tile_m / g.tiles_w) % g.tiles_h) * g.th + (r0 / g.tw) % g.th;
          const int n = (tile_m / (g.tiles_w * g.tiles_h)) * g.tn + r0 / (g.tw * g.th);
          sx1 = w * g.out_mul + g.out_off_w;
          sx2 = h * g.out_mul + g.out_off_h;
          sx3 = n;
          box_in = n < g.batch && h < g.grid_h && w < g.grid_w && sx1 < g.out_w && sx2 < g.out_h;
        } else {
          sx1 = tile_m * BM + r0;
          box_in = sx1 < p.M;
        }
      }
      uint8_t* stage_pre = epi_stage + (warp - 2) * 4096;
      uint8_t* stage_out = stage_pre + 2048;
      if (!mbar_wait(&tmem_full[acc], acc_phase)) { ok = false; break; }
      fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(lane_group * 32) << 16) + (MH == 2 ? second * BN : acc * BN);
      // fused cross-entropy statistics: running (maximum, sum of exp relative to it) of this thread's row over the
      // columns of the tile half it owns, and the target column's logit when it falls into them
      float ce_max = -INFINITY, ce_sum = 0.0f, ce_tl = 0.0f;
      bool ce_hit = false;
      int ce_tgt = -1;
      if constexpr (CE) {
        if (p.ce_mode == 1 && roff >= 0) ce_tgt = (int)p.ce_targets[roff / p.ldd];
      }
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        const int n0 = tile_n * BN + c0;
        uint4 cur[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) cur[q] = aux[q];
        if (c0 + 32 < c_end) gemm_epi::aux_prefetch(aux_row, n0 + 32, p.N, aux);
        tmem_ld_wait();
        if (n0 >= p.N) continue;                               // the same for the whole warp
        const bool tma_chunk = !CE && p.tma_store != 0 && n0 + 32 <= p.N;   // (the launcher rules out split-K here)
        if (!tma_chunk && roff < 0) continue;
        if constexpr (CE) {
          if (p.ce_mode == 1) {
            float cm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.ce_vocab) cm = fmaxf(cm, __uint_as_float(r[j]) * p.alpha);
            if (cm > -INFINITY) {
              const float nm = fmaxf(ce_max, cm);
              float add = 0.0f;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float vj = __uint_as_float(r[j]) * p.alpha;
                if (n0 + j < p.ce_vocab) add += __expf(vj - nm);
                if (n0 + j == ce_tgt) { ce_tl = vj; ce_hit = true; }
              }
              ce_sum = ce_sum * __expf(ce_max - nm) + add;      // exp(-inf) = 0 on the first chunk
              ce_max = nm;
            }
            continue;
          }
        }
        if (p.split_workspace != nullptr) {
          // partial sums of this K split: plain vector stores into the split's slab (zeros for an empty range)
          float* out = p.split_workspace + (long long)wk.split * p.split_stride + roff + n0;
          const bool empty = wk.k_end <= wk.k_begin;
          if (n0 + 32 <= p.N && (p.ldd % 4 == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(out + j) =
                  empty ? make_float4(0, 0, 0, 0)
                        : make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                      __uint_as_float(r[j + 3]));
          } else {
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N) out[j] = empty ? 0.0f : __uint_as_float(r[j]);
          }
          continue;
        }
        if (wk.k_end <= wk.k_begin) continue;
        if constexpr (!CE) {
          if (tma_chunk) {
            // A staging buffer is free once the copy that read it is done (tracked by lane 0, which issued it).
            // Without preact_out the two buffers take turns (stage_turn counts this warp's stored chunks across tiles), so
            // only the copy before the previous one has to be done.
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
        }
        gemm_epi::store_chunk<CE, true>(p, roff, n0, r, cur);
      }
      if constexpr (CE) {
        if (p.ce_mode == 1 && roff >= 0) {
          const long long m = roff / p.ldd;
          const int slot = tile_n * 2 + (MH == 2 ? 0 : second);
          float* dst = p.ce_partial + (m * p.ce_slots + slot) * 2;
          dst[0] = ce_max;
          dst[1] = ce_sum;
          if (ce_hit) p.ce_tgt_logit[m] = ce_tl;
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (MH == 2) { acc_phase ^= 1; }
      else if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0) atomicExch(p.status, GEMM_ERR_EPILOGUE_TIMEOUT);
    if (lane == 0) bulk_wait_group_all();     // this warp's TMA stores have left shared memory and reached global memory
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

// 2-D bf16 matrix [rows, cols] with row pitch `ld` elements; box = 64 columns x `box_rows` rows.
int encode_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return GEMM_ERR_DRIVER;
  fbam_bind_context_to_thread();
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return GEMM_ERR_ALIGNMENT;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, ELEM_TMAP, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_fbam_last_driver_error = (int)r;
  return r == CUDA_SUCCESS ? 0 : GEMM_ERR_TENSORMAP;
}

// NHWC bf16 tensor [n, h, w, c]; box = 64 channels x (tw, th, tn) pixels visited with `stride`.
int encode_nhwc(CUtensorMap* map, const void* base, int n, int h, int w, int c, int tn, int th, int tw, int stride) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return GEMM_ERR_DRIVER;
  fbam_bind_context_to_thread();
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (c * 2) % 16) return GEMM_ERR_ALIGNMENT;
  cuuint64_t dims[4] = {(cuuint64_t)c, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)c * 2, (cuuint64_t)w * c * 2, (cuuint64_t)h * w * c * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)((tw - 1) * stride + 1), (cuuint32_t)((th - 1) * stride + 1), (cuuint32_t)tn};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  CUresult r = enc(map, ELEM_TMAP, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : GEMM_ERR_TENSORMAP;
}

int g_num_sms = 0;

template <int BM, int BN, bool CE = false>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
  using L = SmemLayout<BM, BN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_kernel<BM, BN, CE>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) !=
        cudaSuccess)
      return GEMM_ERR_LAUNCH;
    configured = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = p.tiles_m * ((p.N + BN - 1) / BN) * p.splits;
  const int usable = g_num_sms - g_fbam_reserved_sms > 0 ? g_num_sms - g_fbam_reserved_sms : 1;
  int grid = tiles < usable ? tiles : usable;
  if (p.max_ctas > 0 && grid > p.max_ctas) grid = p.max_ctas;
  CUtensorMap md, mpre;
  p.tma_store = 0;
  std::memset(&md, 0, sizeof(md));
  std::memset(&mpre, 0, sizeof(mpre));
  if (!CE && p.ce_mode == 0 && p.splits <= 1 && p.split_workspace == nullptr && p.mode != GEMM_MODE_WGRAD) {
    const int e = fbam_encode_out_maps(get_encode_fn(), &md, &mpre, p);
    if (e) return e;
  }
  gemm_kernel<BM, BN, CE><<<grid, kThreads, L::kTotal, stream>>>(ma, mb, md, mpre, p);
  return cudaGetLastError() == cudaSuccess ? 0 : GEMM_ERR_LAUNCH;
}

int dispatch(int bm, int bn, const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t s) {
  if (p.ce_mode != 0) return launch<128, 256, true>(ma, mb, p, s);   // the launcher fixed the tile to 128 x 256
  if (bm == 256) {
    if (bn == 128) return launch<256, 128>(ma, mb, p, s);
    return launch<256, 256>(ma, mb, p, s);
  }
  if (bn == 64) return launch<128, 64>(ma, mb, p, s);
  if (bn == 128) return launch<128, 128>(ma, mb, p, s);
  return launch<128, 256>(ma, mb, p, s);
}

// Tall tiles pay off once there are enough of them to fill the machine about twice over.
int pick_bm(long long m, int n, int bn, int requested) {
  if (requested == 128 || requested == 256) return (requested == 256 && bn < 128) ? 128 : requested;
  if (bn < 128) return 128;
  const long long tiles256 = ((m + 255) / 256) * ((n + bn - 1) / bn);
  return tiles256 >= 2 * 148 ? 256 : 128;
}

int pick_bn(int n, int requested) {
  if (requested == 64 || requested == 128 || requested == 256) return requested;
  if (n <= 64) return 64;
  if (n <= 128) return 128;
  return 256;
}

}  // namespace

// A persistent kernel sized to the whole machine cannot finish while another long-running kernel (a library
// send/receive that waits for its peer, say) occupies some SMs: its last CTAs are never scheduled.  Callers that
// keep such kernels in flight reserve SMs for them; every persistent GEMM / convolution launch then uses at most
// (SM count - n) CTAs.  Returns the previous value.
// Driver result code of the most recent failed tensor-map encode, and the runtime's pending error (not cleared).
extern "C" int fbam_last_driver_error() { return g_fbam_last_driver_error; }
extern "C" int fbam_pending_runtime_error() { return (int)cudaPeekAtLastError(); }

// Layout of GemmParams as this library was compiled: total size, then the offsets of a few fields spread over
// the struct.  Callers that mirror the struct (the ctypes binding) compare these with their own layout at load.
extern "C" void fbam_gemm_params_layout(long long* out) {
  out[0] = (long long)sizeof(GemmParams);
  out[1] = (long long)offsetof(GemmParams, status);
  out[2] = (long long)offsetof(GemmParams, split_workspace);
  out[3] = (long long)offsetof(GemmParams, rs_out);
  out[4] = (long long)offsetof(GemmParams, rs_row_stores);
  out[5] = (long long)offsetof(GemmParams, mode);
  out[6] = (long long)offsetof(GemmParams, conv);
  out[7] = (long long)sizeof(ConvGeom);
}

// 1 when this library was compiled with IEEE half elements, 0 for bf16 (see elem16.cuh).
extern "C" int fbam_elem_is_fp16() { return ELEM_IS_FP16; }

// 1 when the row-store variant of the reduce-scatter epilogue was compiled in (see gemm_epilogue.cuh).
extern "C" int fbam_has_rs_row_stores() { return FBAM_RS_ROW_STORES; }

extern "C" int fbam_set_reserved_sms(int n) {
  const int old = g_fbam_reserved_sms;
  g_fbam_reserved_sms = n < 0 ? 0 : n;
  return old;
}

extern "C" int fbam_gemm(const void* A, long long lda, int a_mn_major, const void* B, long long ldb,
                              int b_mn_major, int M, int N, int K, GemmParams* params, void* stream) {
  GemmParams p = *params;
  if (M <= 0 || N <= 0 || K <= 0) return GEMM_ERR_SHAPE;
  p.mode = GEMM_MODE_PLAIN;
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.k_blocks = (K + BK - 1) / BK;
  if (p.splits < 1) p.splits = 1;
  if (p.splits > p.k_blocks) p.splits = p.k_blocks;
  if (p.splits > 1 && p.split_workspace == nullptr && !(p.out_fp32 && p.accumulate == GEMM_ACC_ATOMIC))
    return GEMM_ERR_SHAPE;
  int bn = pick_bn(N, p.bn);
  int BM = pick_bm(M, N, bn, p.bm);
  if (p.ce_mode != 0) {
    // fused cross-entropy epilogues: one tile shape, no split-K, the buffers of the mode present
    if (p.ce_mode < 0 || p.ce_mode > 2 || p.splits != 1 || p.ce_targets == nullptr || p.ce_vocab < 1 || p.ce_vocab > N)
      return GEMM_ERR_SHAPE;
    bn = 256;
    BM = 128;
    if (p.ce_mode == 1 && (p.ce_partial == nullptr || p.ce_tgt_logit == nullptr || p.ce_slots != 2 * ((N + bn - 1) / bn)))
      return GEMM_ERR_SHAPE;
    if (p.ce_mode == 2 && (p.ce_lse == nullptr || p.D == nullptr)) return GEMM_ERR_SHAPE;
    if (p.ce_mode == 1 && p.ldd <= 0) return GEMM_ERR_SHAPE;       // ldd only turns row offsets back into rows
  }
  p.tiles_m = (M + BM - 1) / BM;
  const int elt = p.out_fp32 ? 4 : 2;
  p.vec_ok = (p.ldd % (16 / elt) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
             (p.preact_out == nullptr || (reinterpret_cast<uintptr_t>(p.preact_out) & 15) == 0) &&
             (p.gelu_grad_in == nullptr || (reinterpret_cast<uintptr_t>(p.gelu_grad_in) & 15) == 0) &&
             (p.residual == nullptr || (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0) && (p.ldd % 8 == 0);
  if (p.rs_rows_per_rank > 0) {
    if (p.mode != GEMM_MODE_PLAIN) return GEMM_ERR_SHAPE;
    p.vec_ok = (p.ldd % (p.rs_slot_plus1 > 0 ? 8 : 4) == 0);
    for (int r = 0; r * p.rs_rows_per_rank < M; ++r)
      if (r >= 8 || p.rs_out[r] == nullptr || (reinterpret_cast<uintptr_t>(p.rs_out[r]) & 15)) return GEMM_ERR_ALIGNMENT;
  }
  if (p.ready_flags != nullptr && (p.flag_rows <= 0)) return GEMM_ERR_SHAPE;
  if (p.flag_spin_limit == 0) p.flag_spin_limit = 1u << 22;
  CUtensorMap ma, mb;
  int e;
  if (a_mn_major) e = encode_2d(&ma, A, K, M, lda, 64);  // rows = K, cols = M, panels of 64 columns
  else e = encode_2d(&ma, A, M, K, lda, BM);  // one box of BM rows
  if (e) return e;
  if (b_mn_major) e = encode_2d(&mb, B, K, N, ldb, 64);
  else e = encode_2d(&mb, B, N, K, ldb, bn);
  if (e) return e;
  return dispatch(BM, bn, ma, mb, p, reinterpret_cast<cudaStream_t>(stream));
}

// Implicit-GEMM convolution pass.  `X` is the gathered NHWC tensor [batch, in_h, in_w, C]; `Wmat` is the
// filter matrix [N, taps*C] (K-major; tap-major then channel).  See ConvGeom for the tiling fields.
extern "C" int fbam_conv(const void* X, int in_h, int in_w, int C, const void* Wmat, long long ldw, int N,
                              GemmParams* params, void* stream) {
  GemmParams p = *params;
  if (p.num_classes != 0) return GEMM_ERR_SHAPE;   // fused parity classes exist in the CTA-pair kernel only
  ConvGeom& g = p.conv;
  const int BM = g.tn * g.th * g.tw;
  if (C % 64 != 0 || (BM != 128 && BM != 256) || g.num_taps < 1 || g.num_taps > 9) return GEMM_ERR_SHAPE;
  p.mode = GEMM_MODE_CONV;
  p.a_mn_major = 0; p.b_mn_major = 0;
  g.c_blocks = C / 64;
  g.tiles_w = (g.grid_w + g.tw - 1) / g.tw;
  g.tiles_h = (g.grid_h + g.th - 1) / g.th;
  const int tiles_nb = (g.batch + g.tn - 1) / g.tn;
  p.tiles_m = g.tiles_w * g.tiles_h * tiles_nb;
  p.M = p.tiles_m * BM;
  p.N = N; p.K = g.num_taps * C;
  p.k_blocks = g.num_taps * g.c_blocks;
  p.splits = 1;
  const int bn = pick_bn(N, p.bn);
  if (BM == 256 && bn < 128) return GEMM_ERR_SHAPE;
  const int elt = p.out_fp32 ? 4 : 2;
  p.vec_ok = (p.ldd % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) && (p.ldd % (16 / elt) == 0);
  CUtensorMap ma, mb;
  int e = encode_nhwc(&ma, X, g.batch, in_h, in_w, C, g.tn, g.th, g.tw, g.in_mul);
  if (e) return e;
  e = encode_2d(&mb, Wmat, N, p.K, ldw, bn);
  if (e) return e;
  return dispatch(BM, bn, ma, mb, p, reinterpret_cast<cudaStream_t>(stream));
}

// Convolution weight gradient as a split-K GEMM over output pixels:
//   dW[o, tap, c] += sum_pixels dY[pixel, o] * X[gather(pixel, tap), c]
// dY: NHWC [batch, out_h, out_w, O]; X: NHWC [batch, in_h, in_w, C]; dW: fp32 [O, taps*C], must be zeroed by
// the caller (CTAs add their partial sums atomically).  conv.{tn,th,tw} describe the 64-pixel K brick.
extern "C" int fbam_conv_wgrad(const void* dY, int O, const void* X, int in_h, int in_w, int C,
                                    GemmParams* params, void* stream) {
  GemmParams p = *params;
  ConvGeom& g = p.conv;
  if (C % 64 != 0 || O % 8 != 0 || g.tn * g.th * g.tw != BK || g.num_taps < 1 || g.num_taps > 9) return GEMM_ERR_SHAPE;
  if (!p.out_fp32) return GEMM_ERR_SHAPE;
  p.mode = GEMM_MODE_WGRAD;
  p.a_mn_major = 1; p.b_mn_major = 1;
  p.accumulate = GEMM_ACC_ATOMIC;
  g.c_blocks = C / 64;
  g.tiles_w = (g.grid_w + g.tw - 1) / g.tw;
  g.tiles_h = (g.grid_h + g.th - 1) / g.th;
  const int bricks = g.tiles_w * g.tiles_h * ((g.batch + g.tn - 1) / g.tn);
  p.M = O; p.N = g.num_taps * C; p.K = bricks * BK;
  // N tiles may span two filter taps (each 64-column panel is gathered with its own tap), so 256-wide tiles
  // work for every C that is a multiple of 64.
  int bn = p.N >= 256 ? 256 : (p.N >= 128 ? 128 : 64);
  if (p.bn == 64 || p.bn == 128 || p.bn == 256) bn = p.bn;
  const int BM = (O >= 256 && bn >= 128 && p.bm != 128) ? 256 : 128;
  p.tiles_m = (O + BM - 1) / BM;
  p.k_blocks = bricks;
  if (p.splits < 1) {
    if (g_num_sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int tiles = p.tiles_m * ((p.N + bn - 1) / bn);
    p.splits = (g_num_sms + tiles - 1) / tiles;
  }
  if (p.splits > bricks) p.splits = bricks;
  p.vec_ok = 0;
  CUtensorMap ma, mb;
  int e = encode_nhwc(&ma, dY, g.batch, g.grid_h, g.grid_w, O, g.tn, g.th, g.tw, 1);
  if (e) return e;
  e = encode_nhwc(&mb, X, g.batch, in_h, in_w, C, g.tn, g.th, g.tw, g.in_mul);
  if (e) return e;
  return dispatch(BM, bn, ma, mb, p, reinterpret_cast<cudaStream_t>(stream));
}
