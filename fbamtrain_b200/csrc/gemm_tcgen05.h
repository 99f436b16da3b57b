// Parameter blocks of the tcgen05 GEMM / implicit-GEMM convolution entry points.  The Python side
// mirrors these structs field for field with ctypes (fbamtrain_b200/ops/native.py).
#pragma once
#include "elem16.cuh"
#include <stdint.h>

enum { GEMM_MODE_PLAIN = 0, GEMM_MODE_CONV = 1, GEMM_MODE_WGRAD = 2 };
enum { GEMM_ACT_NONE = 0, GEMM_ACT_GELU = 1, GEMM_ACT_RELU = 2 };
enum { GEMM_ACC_NONE = 0, GEMM_ACC_RMW = 1, GEMM_ACC_ATOMIC = 2 };
enum {
  GEMM_ERR_SHAPE = 1, GEMM_ERR_ALIGNMENT = 2, GEMM_ERR_TENSORMAP = 3, GEMM_ERR_DRIVER = 4, GEMM_ERR_LAUNCH = 5,
  GEMM_ERR_PRODUCER_TIMEOUT = 101, GEMM_ERR_MMA_TIMEOUT = 102, GEMM_ERR_EPILOGUE_TIMEOUT = 103
};

// Geometry of one implicit-GEMM convolution pass.  The 128 rows of an output tile are a brick of
// tn x th x tw positions of a (batch, grid_h, grid_w) iteration grid.  Grid position (h, w) gathers
// input pixel (h*in_mul + tap_dh[t], w*in_mul + tap_dw[t]) for tap t and writes output pixel
// (h*out_mul + out_off_h, w*out_mul + out_off_w) of an (out_h, out_w) image.
struct ConvGeom {
  int batch, grid_h, grid_w;
  int tn, th, tw;
  int in_mul;
  int out_mul, out_off_h, out_off_w, out_h, out_w;
  int num_taps;
  int tap_dh[9], tap_dw[9];
  // derived by the launcher
  int c_blocks, tiles_w, tiles_h;
};

// One parity class of a strided data-gradient convolution run by the CTA-pair kernel as part of a fused pass: its own
// taps, its own output offset, and where its filter columns start in the shared filter matrix (in 64-column blocks).
struct ConvClass {
  int num_taps;
  int tap_dh[4], tap_dw[4];
  int out_off_h, out_off_w;
  int k_block_base;
};

struct GemmParams {
  void* D;                          // output, bf16 or fp32, row pitch ldd elements
  long long ldd;
  const void* bias;                 // [N] or null
  const elem_t* residual;    // [M, N] pitch ldr, added after the activation, or null
  long long ldr;
  elem_t* preact_out;        // [M, N] pitch ldd: value before the activation, or null
  const elem_t* gelu_grad_in;  // [M, N] pitch ldd: result is multiplied by gelu'(this), or null
  int* status;                      // device word, receives an error code on a timed-out wait
  float alpha;
  int out_fp32, bias_fp32, act, accumulate;
  int bn;                           // 0 = choose from N; else 64 / 128 / 256
  int bm;                           // 0 = choose from the tile count; else 128 / 256 (plain GEMM and wgrad)
  int max_ctas;                     // 0 = one per SM
  int splits;                       // split-K factor (needs fp32 output with atomic accumulation); 0/1 = none
  // split-K without atomics: split s writes its partial tile to split_workspace + s * split_stride (fp32,
  // same pitch as D) with plain stores; the caller sums the partials afterwards
  float* split_workspace;
  long long split_stride;
  // all-gather -> GEMM: rows of the gated operand arrive from peers; rows [i*flag_rows, (i+1)*flag_rows) are
  // complete once ready_flags[i] >= flag_epoch (ready_flags is in local memory; peers store to it)
  const unsigned* ready_flags;
  int tile_m_rotate;                // tile rows are visited starting at this tile index (own shard first)
  int flag_rows, flag_on_b;
  unsigned flag_epoch, flag_spin_limit;
  // GEMM -> reduce-scatter: fp32 partial sums are added (system-scope reductions over peer memory) into the
  // buffer of the rank that owns the output row: owner = m / rs_rows_per_rank, local row = m % rs_rows_per_rank
  void* rs_out[8];
  int rs_rows_per_rank;
  // rs_slot_plus1 = 0: the mode above.  rs_slot_plus1 = s + 1: instead of adding, the tile is rounded to bf16 and
  // written with plain vector stores into slot s of the owner's buffer, laid out [slot][rs_rows_per_rank][ldd]
  // (one slot per source rank); the owner sums the slots afterwards.  Plain stores run at link bandwidth, remote
  // reductions do not.
  int rs_slot_plus1;
  // rs_row_stores != 0 (slot form only): the four lanes that hold four neighbouring rows exchange their 16-byte
  // pieces first, so that one store instruction writes 64 contiguous bytes of a row (two full sectors per
  // NVLink write) instead of 16 bytes of each of 32 rows.  Needs M and rs_rows_per_rank to be multiples of 32.
  int rs_row_stores;
  // Fused LM head + cross-entropy (plain GEMM on single CTAs with 128 x 256 tiles): the logits tile stays in tensor
  // memory / registers and never reaches HBM as fp32.
  //   ce_mode 1 (statistics): nothing is stored per element.  Every epilogue thread reduces its row's columns of the
  //     tile half it owns to (maximum, sum of exp relative to that maximum) and writes the pair to
  //     ce_partial[(row * ce_slots + slot) * 2 + {0, 1}], slot = tile_n * 2 + column half; the thread that meets the
  //     row's target column writes that logit to ce_tgt_logit[row].  Columns >= ce_vocab are padding and ignored.
  //   ce_mode 2 (gradient): the value stored to D is ce_scale * (exp(logit - ce_lse[row]) - [column == target]);
  //     padding columns get 0.
  int ce_mode, ce_vocab, ce_slots;
  float ce_scale;
  float* ce_partial;
  float* ce_tgt_logit;
  const float* ce_lse;
  const long long* ce_targets;
  // filled by the launcher
  int mode, M, N, K, tiles_m, k_blocks, a_mn_major, b_mn_major, vec_ok;
  ConvGeom conv;
  // Fused parity classes (CTA-pair convolution only; 0 = a single pass with conv's own taps and offset).  Every
  // 256-row tile is computed num_classes times in a row by the same CTA pair, once per class, each time with that
  // class's taps, filter columns and output offset: the input tile is fetched from DRAM once and found in L2 by the
  // other classes, instead of being streamed again by a separate launch per class.
  int num_classes;
  ConvClass cls[4];
  // Filled by the CTA-pair launchers.  tma_store: 0 = the epilogue stores from registers; 1 = 16-bit results leave
  // through shared memory and TMA tiled stores (D only); 2 = D and preact_out.  st_bw / st_bh / st_bn: the 32 rows
  // that one epilogue warp owns, as a box of output positions (w, h, n) of a convolution brick (1, 1, 32 rows of a
  // plain matrix).
  int tma_store, st_bw, st_bh, st_bn;
};

// Driver entry points (tensor-map encoding) need a context that is current on the CALLING thread.  A thread that
// has only inherited "device 0" by default (an autograd worker whose first CUDA work is one of these launchers)
// has none yet; a runtime call that names the device binds the primary context to it.
static inline void fbam_bind_context_to_thread() {
  static thread_local int bound = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev != bound) {
    cudaSetDevice(dev);
    bound = dev;
  }
}

