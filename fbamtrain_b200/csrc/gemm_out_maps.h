// Tensor maps for the epilogue's TMA stores, shared by the single-CTA and the CTA-pair launchers.
#pragma once
#include <cuda.h>
#include <cstring>
#include <stdint.h>

#include "gemm_tcgen05.h"

extern int g_fbam_last_driver_error;   // defined in gemm_tcgen05.cu

// Tensor maps of the output (and of preact_out) for the epilogue's TMA stores: boxes of 32 columns x the 32 rows of one
// epilogue warp, 64-byte swizzle (the layout gemm_epi::stage_row64 writes).  Returns 0 when the stores cannot take this
// route (fp32 output, accumulation, reduce-scatter forms, unaligned output) and leaves tma_store at 0.
template <typename EncFn>
static inline int fbam_encode_out_maps(EncFn enc, CUtensorMap* md, CUtensorMap* mpre, GemmParams& p) {
  p.tma_store = 0;
  p.st_bw = p.st_bh = 1;
  p.st_bn = 32;
  std::memset(md, 0, sizeof(CUtensorMap));
  std::memset(mpre, 0, sizeof(CUtensorMap));
  if (p.out_fp32 || p.accumulate != 0 || p.rs_rows_per_rank > 0 || !p.vec_ok || p.N < 32 || (p.ldd * 2) % 16 != 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p.D) & 15) || (p.preact_out && (reinterpret_cast<uintptr_t>(p.preact_out) & 15))) return 0;
  if (!enc) return GEMM_ERR_DRIVER;
  fbam_bind_context_to_thread();
  CUresult r1 = CUDA_SUCCESS, r2 = CUDA_SUCCESS;
  if (p.mode == GEMM_MODE_CONV) {
    const ConvGeom& g = p.conv;
    // tiles are padded to whole bricks; the register path skips positions outside the iteration grid, the copy only
    // clips at the edge of the output: take this route only when the first position outside the grid also lies
    // outside the output, for every output offset in use
    const int n_off = p.num_classes > 0 ? p.num_classes : 1;
    for (int c = 0; c < n_off; ++c) {
      const int oh = p.num_classes > 0 ? p.cls[c].out_off_h : g.out_off_h;
      const int ow = p.num_classes > 0 ? p.cls[c].out_off_w : g.out_off_w;
      if (g.grid_h * g.out_mul + oh < g.out_h || g.grid_w * g.out_mul + ow < g.out_w || oh < 0 || ow < 0) return 0;
    }
    if (g.tw > 32 ? g.tw % 32 != 0 : 32 % g.tw != 0) return 0;
    const int bw = g.tw < 32 ? g.tw : 32;
    const int rest = 32 / bw;
    if (g.th > rest ? g.th % rest != 0 : rest % g.th != 0) return 0;
    const int bh = g.th < rest ? g.th : rest;
    const int bn = 32 / (bw * bh);
    if (bn > g.tn || g.tn % bn != 0) return 0;
    p.st_bw = bw; p.st_bh = bh; p.st_bn = bn;
    cuuint64_t dims[4] = {(cuuint64_t)p.N, (cuuint64_t)g.out_w, (cuuint64_t)g.out_h, (cuuint64_t)g.batch};
    cuuint64_t strides[3] = {(cuuint64_t)p.ldd * 2, (cuuint64_t)g.out_w * p.ldd * 2,
                             (cuuint64_t)g.out_h * g.out_w * p.ldd * 2};
    cuuint32_t box[4] = {32, (cuuint32_t)((bw - 1) * g.out_mul + 1), (cuuint32_t)((bh - 1) * g.out_mul + 1), (cuuint32_t)bn};
    cuuint32_t estr[4] = {1, (cuuint32_t)g.out_mul, (cuuint32_t)g.out_mul, 1};
    r1 = enc(md, ELEM_TMAP, 4, p.D, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (p.preact_out)
      r2 = enc(mpre, ELEM_TMAP, 4, p.preact_out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[2] = {(cuuint64_t)p.N, (cuuint64_t)p.M};
    cuuint64_t strides[1] = {(cuuint64_t)p.ldd * 2};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    r1 = enc(md, ELEM_TMAP, 2, p.D, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (p.preact_out)
      r2 = enc(mpre, ELEM_TMAP, 2, p.preact_out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r1 != CUDA_SUCCESS || r2 != CUDA_SUCCESS) {
    g_fbam_last_driver_error = (int)(r1 != CUDA_SUCCESS ? r1 : r2);
    return GEMM_ERR_TENSORMAP;
  }
  p.tma_store = p.preact_out ? 2 : 1;
  return 0;
}

