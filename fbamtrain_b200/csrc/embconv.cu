// Cell embedding fused with the first convolution of the frame head.
//
// The cell embedding is linear in three small tables (code-point rows, position rows, six colour vectors) and a
// convolution without a normalisation in front of it is linear in its input, so the pre-activation of the first
// convolution is a sum of table look-ups:
//
//   Z[n, p, :] = sum_taps T[cp(n, cell(p, tap))][tap][:]            code points:  T[v][tap] = cp_embed[v] . W[:, tap, :]^T
//              + POS[p][:]                                         positions:    the convolution of the position table
//              + sum_taps sum_c (rgb_c / 255) . CC[tap][c][:]      colours:      CC[tap][c] = colour[c] . W[:, tap, :]^T
//
// and its backward needs only three reductions of dZ: by (code point, tap), over the frames, and colour-weighted.
// The (frames x cells x channels) embedding tensor, the data-gradient convolution into it and its scatter into the
// tables are never computed.  What the reference does with build_cell_embeds + conv2d and their backward kernels
// (kernel_gen/kernel_gen/kernels/build_cell_embeds.py:74-134, build_cell_embeds_bwd.py:6-322,
// src/framehead_model.cpp:126-175, 601-731) is covered here by
//
//   fbam_embconv_features    colour features F[n, p, tap*6 + c] = rgb_c(cell(p, tap)) / 255 (bf16, 64 per pixel):
//                            the colour term is the GEMM F . CC (forward) and F^T . dZ (backward) on the tensor cores
//   fbam_embconv_fwd         Z += POS + table rows; Y = GELU(Z)
//   fbam_embconv_bwd_reduce  S[v][tap][:] += dZ rows by code point and tap;  D[p][:] += dZ summed over frames
//
// A warp owns one output pixel (32 lanes x 8 channels = a 256-channel block) and walks a run of consecutive frames.
// Terminal frames change little from one frame to the next, and both kernels use that without depending on it:
// the forward kernel keeps the sum of the nine table rows and, when a few of the nine code points changed, subtracts
// the old rows and adds the new ones (it rebuilds the sum from scratch when more than four changed and at the start
// of every run, which also bounds the rounding drift); the backward kernel accumulates dZ in registers per tap
// while that tap's code point stays the same and adds the run to S with vector reductions only when it changes.
// Frames that share nothing cost nine row loads (forward) or nine row reductions (backward) per pixel and frame.
#include "elem16.cuh"
#include <cuda_runtime.h>
#include <stdint.h>

#include "gelu_math.cuh"

namespace {


struct EmbConvGeom {
  int rows, cols;        // cells per frame
  int oh, ow;            // output pixels per frame
  int stride, pad, dil;  // 3x3 filter geometry
};

struct alignas(16) Pack8 { elem2_t h[4]; };
// Cell index (row-major within the frame) that output pixel (oy, ox) reads through filter tap `tap`, or -1 when the
// tap falls into the padding.
__device__ __forceinline__ int tap_cell(const EmbConvGeom& g, int oy, int ox, int tap) {
  const int iy = oy * g.stride + (tap / 3) * g.dil - g.pad;
  const int ix = ox * g.stride + (tap % 3) * g.dil - g.pad;
  if (iy < 0 || iy >= g.rows || ix < 0 || ix >= g.cols) return -1;
  return iy * g.cols + ix;
}

// ------------------------------------------------------------------------------------------------
// colour features: one thread per output pixel writes its 128-byte row
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embconv_features_kernel(const int* __restrict__ cells, elem_t* __restrict__ feat,
                                                               long long frames, EmbConvGeom g) {
  const int p_out = g.oh * g.ow;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= frames * p_out) return;
  const long long n = idx / p_out;
  const int p = (int)(idx % p_out);
  const int oy = p / g.ow, ox = p % g.ow;
  const long long frame_base = n * (long long)(g.rows * g.cols);
  uint32_t w[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) w[i] = 0u;
#pragma unroll
  for (int t = 0; t < 9; ++t) {
    const int cell = tap_cell(g, oy, ox, t);
    if (cell >= 0) {
      const int* cw = cells + (frame_base + cell) * 3;
      const uint32_t fg = (uint32_t)__ldg(cw + 1), bg = (uint32_t)__ldg(cw + 2);
      const float k = 1.0f / 255.0f;
      const elem2_t a = ff2e2(((fg >> 16) & 255) * k, ((fg >> 8) & 255) * k);
      const elem2_t b = ff2e2((fg & 255) * k, ((bg >> 16) & 255) * k);
      const elem2_t c = ff2e2(((bg >> 8) & 255) * k, (bg & 255) * k);
      w[t * 3 + 0] = *reinterpret_cast<const uint32_t*>(&a);
      w[t * 3 + 1] = *reinterpret_cast<const uint32_t*>(&b);
      w[t * 3 + 2] = *reinterpret_cast<const uint32_t*>(&c);
    }
  }
  uint4* dst = reinterpret_cast<uint4*>(feat + idx * 64);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

// ------------------------------------------------------------------------------------------------
// forward: Z += POS + sum of table rows, Y = GELU(Z)
// ------------------------------------------------------------------------------------------------
constexpr int kPrefetch = 4;       // frames whose cell words / rows are fetched before any of them is used (forward)
constexpr int kPrefetchBwd = 16;   // same in the backward reduction (8-byte pieces: 128 bytes in flight per lane)

using gelu_math::f2;
using gelu_math::gelu2;

__device__ __forceinline__ void add_row(float2* acc, const elem_t* row, float sign) {
  const Pack8 r = *reinterpret_cast<const Pack8*>(row);
  const float2 s2 = f2(sign);
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j] = __ffma2_rn(s2, e22ff(r.h[j]), acc[j]);
}

__global__ void __launch_bounds__(256, 3) embconv_fwd_kernel(const int* __restrict__ cells, const elem_t* __restrict__ table,
                                                             const float* __restrict__ pos, elem_t* __restrict__ z,
                                                             elem_t* __restrict__ y, long long frames, int vocab, int O,
                                                             EmbConvGeom g, int seg_len, int nseg, int z_has_input,
                                                             int apply_gelu) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const int p_out = g.oh * g.ow;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)p_out * nseg) return;             // the whole warp leaves together
  const int seg = (int)(item / p_out), p = (int)(item % p_out);
  const int cell = lane < 9 ? tap_cell(g, p / g.ow, p % g.ow, lane) : -1;
  const int co = blockIdx.y * 256 + lane * 8;
  const bool act = co < O;
  const long long cells_per_frame = (long long)g.rows * g.cols;
  float2 base[4], sum[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) { base[j] = f2(0.0f); sum[j] = f2(0.0f); }
  if (act && pos != nullptr) {
    const float4* pp = reinterpret_cast<const float4*>(pos + (long long)p * O + co);
    const float4 a = pp[0], b = pp[1];
    base[0] = make_float2(a.x, a.y); base[1] = make_float2(a.z, a.w);
    base[2] = make_float2(b.x, b.y); base[3] = make_float2(b.z, b.w);
  }
  int cur = -1;                                            // lanes 0..8: code point of this lane's tap (-1: none)
  const long long f0 = (long long)seg * seg_len;
  const long long f1 = min(frames, f0 + seg_len);
  const long long row9 = 9ll * O;
  const elem_t* tab = table + (act ? co : 0);
  const int* cell_ptr = cells + (f0 * cells_per_frame + max(cell, 0)) * 3;
  const long long cell_step = cells_per_frame * 3, z_step = (long long)p_out * O;
  long long off = (f0 * p_out + p) * O + (act ? co : 0);
  for (long long fb = f0; fb < f1; fb += kPrefetch) {
    int ncp[kPrefetch];
    Pack8 zin[kPrefetch];
#pragma unroll
    for (int u = 0; u < kPrefetch; ++u) {
      ncp[u] = -1;
      if (fb + u < f1) {
        if (cell >= 0) ncp[u] = __ldg(cell_ptr + u * cell_step);
        if (act && z_has_input) zin[u] = *reinterpret_cast<const Pack8*>(z + off + u * z_step);
      }
    }
    cell_ptr += kPrefetch * cell_step;
#pragma unroll
    for (int u = 0; u < kPrefetch; ++u) {
      const long long f = fb + u;
      if (f >= f1) break;
      int nc = ncp[u];
      if ((unsigned)nc >= (unsigned)vocab) nc = -1;        // outside the table (or padding): contributes nothing
      const unsigned changed = __ballot_sync(full, nc != cur) & 0x1ffu;
      if (f == f0 || __popc(changed) > 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) sum[j] = f2(0.0f);
#pragma unroll
        for (int t = 0; t < 9; ++t) {
          const int c = __shfl_sync(full, nc, t);
          if (c >= 0 && act) add_row(sum, tab + c * row9 + t * O, 1.0f);
        }
      } else {
        unsigned m = changed;
        while (m) {
          const int t = __ffs(m) - 1;
          m &= m - 1;
          const int o = __shfl_sync(full, cur, t);
          const int c = __shfl_sync(full, nc, t);
          if (act) {
            if (o >= 0) add_row(sum, tab + o * row9 + t * O, -1.0f);
            if (c >= 0) add_row(sum, tab + c * row9 + t * O, 1.0f);
          }
        }
      }
      cur = nc;
      if (act) {
        float2 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[j] = __fadd2_rn(sum[j], base[j]);
          if (z_has_input) v[j] = __fadd2_rn(v[j], e22ff(zin[u].h[j]));
        }
        Pack8 out;
#pragma unroll
        for (int j = 0; j < 4; ++j) out.h[j] = f22e2(v[j]);
        *reinterpret_cast<Pack8*>(z + off + u * z_step) = out;
        if (y != nullptr) {
          if (apply_gelu) {
#pragma unroll
            for (int j = 0; j < 4; ++j) out.h[j] = f22e2(gelu2(v[j]));
          }
          *reinterpret_cast<Pack8*>(y + off + u * z_step) = out;
        }
      }
    }
    off += kPrefetch * z_step;
  }
}

// ------------------------------------------------------------------------------------------------
// backward: S[v][tap][:] += dZ rows whose tap shows code point v;  D[p][:] += sum over frames of dZ[:, p, :]
// ------------------------------------------------------------------------------------------------
// A lane owns 4 channels (a warp covers a 128-channel block).  All nine taps of a pixel accumulate the same dZ
// values and differ only in where their runs begin and end, so the lane keeps ONE running prefix sum of its dZ over
// the frames of the segment and, per tap, the value of that prefix when the tap's current run began: a run's sum is
// the difference of two prefixes, taken when the run ends.  Per frame that is four additions instead of forty; the
// prefix at the end of the segment is the pixel's contribution to D.  (The prefix spans at most one segment, so the
// difference loses at most log2(segment) bits of fp32 — far below the bf16 resolution of dZ.)
struct alignas(8) Pack4 { elem2_t h[2]; };

__device__ __forceinline__ void red_add4(float* dst, float4 v) { atomicAdd(reinterpret_cast<float4*>(dst), v); }

__global__ void __launch_bounds__(256, 3) embconv_bwd_reduce_kernel(const int* __restrict__ cells, const elem_t* __restrict__ dz,
                                                                    float* __restrict__ S, float* __restrict__ D,
                                                                    long long frames, int vocab, int O, EmbConvGeom g,
                                                                    int seg_len, int nseg) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const int p_out = g.oh * g.ow;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)p_out * nseg) return;
  const int seg = (int)(item / p_out), p = (int)(item % p_out);
  const int cell = lane < 9 ? tap_cell(g, p / g.ow, p % g.ow, lane) : -1;
  const int co = blockIdx.y * 128 + lane * 4;
  const bool act = co < O;
  const long long cells_per_frame = (long long)g.rows * g.cols;
  const long long row9 = 9ll * O;
  float2 pre[2] = {f2(0.0f), f2(0.0f)};                     // prefix sum of this lane's dZ over the frames so far
  // per tap: the prefix when its current run began.  Touched only when a run ends, so it lives in shared memory
  // (one 16-byte slot per thread and tap, conflict-free) and the loop over the changed taps is a real loop.
  __shared__ float4 start_sm[9][256];
  float4* start = &start_sm[0][threadIdx.x];
#pragma unroll
  for (int t = 0; t < 9; ++t) start[t * 256] = make_float4(0.f, 0.f, 0.f, 0.f);
  int cur = -1;
  const long long f0 = (long long)seg * seg_len;
  const long long f1 = min(frames, f0 + seg_len);
  const int* cell_ptr = cells + (f0 * cells_per_frame + max(cell, 0)) * 3;
  const elem_t* dz_ptr = dz + (f0 * p_out + p) * O + (act ? co : 0);
  const long long cell_step = cells_per_frame * 3, dz_step = (long long)p_out * O;
  float* s_base = S + (act ? co : 0);
  for (long long fb = f0; fb < f1; fb += kPrefetchBwd) {
    int ncp[kPrefetchBwd];
    Pack4 din[kPrefetchBwd];
#pragma unroll
    for (int u = 0; u < kPrefetchBwd; ++u) {
      ncp[u] = -1;
      if (fb + u < f1) {
        if (cell >= 0) ncp[u] = __ldg(cell_ptr + u * cell_step);
        if (act) din[u] = *reinterpret_cast<const Pack4*>(dz_ptr + u * dz_step);
      }
    }
    cell_ptr += kPrefetchBwd * cell_step;
    dz_ptr += kPrefetchBwd * dz_step;
#pragma unroll
    for (int u = 0; u < kPrefetchBwd; ++u) {
      if (fb + u >= f1) break;
      int nc = ncp[u];
      if ((unsigned)nc >= (unsigned)vocab) nc = -1;
      unsigned changed = __ballot_sync(full, nc != cur) & 0x1ffu;
      while (changed) {
        const int t = __ffs(changed) - 1;
        changed &= changed - 1;
        const int o = __shfl_sync(full, cur, t);
        const float4 st = start[t * 256];
        if (o >= 0 && act)
          red_add4(s_base + o * row9 + t * O, make_float4(pre[0].x - st.x, pre[0].y - st.y, pre[1].x - st.z, pre[1].y - st.w));
        start[t * 256] = make_float4(pre[0].x, pre[0].y, pre[1].x, pre[1].y);
      }
      cur = nc;
      if (act) {
        pre[0] = __fadd2_rn(pre[0], e22ff(din[u].h[0]));
        pre[1] = __fadd2_rn(pre[1], e22ff(din[u].h[1]));
      }
    }
  }
#pragma unroll 1
  for (int t = 0; t < 9; ++t) {
    const int o = __shfl_sync(full, cur, t);
    const float4 st = start[t * 256];
    if (o >= 0 && act)
      red_add4(s_base + o * row9 + t * O, make_float4(pre[0].x - st.x, pre[0].y - st.y, pre[1].x - st.z, pre[1].y - st.w));
  }
  if (act && f1 > f0) red_add4(D + (long long)p * O + co, make_float4(pre[0].x, pre[0].y, pre[1].x, pre[1].y));
}

// ------------------------------------------------------------------------------------------------
// sum of split-K slabs: out[i] = sum_s work[s][i], written as fp32 or bf16
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) slab_reduce_kernel(const float* __restrict__ work, void* __restrict__ out,
                                                          long long n, int slabs, int out_elem) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < slabs; ++k) {
    const float4 v = *reinterpret_cast<const float4*>(work + (long long)k * n + i);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  if (out_elem) {
    elem2_t* o = reinterpret_cast<elem2_t*>(reinterpret_cast<elem_t*>(out) + i);
    o[0] = ff2e2(s.x, s.y);
    o[1] = ff2e2(s.z, s.w);
  } else {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + i) = s;
  }
}

bool geom_ok(const EmbConvGeom& g) {
  if (g.rows < 1 || g.cols < 1 || g.oh < 1 || g.ow < 1 || g.stride < 1 || g.dil < 1 || g.pad < 0) return false;
  // the last output pixel's first tap must not start beyond the frame by more than the padding allows
  const int need_h = (g.oh - 1) * g.stride - g.pad, need_w = (g.ow - 1) * g.stride - g.pad;
  return need_h < g.rows && need_w < g.cols;
}

int launch_result() { return cudaGetLastError() == cudaSuccess ? 0 : 5; }

}  // namespace

// Return codes: 0 ok, 1 unsupported shape, 2 misaligned pointer, 5 launch failure.
extern "C" int fbam_embconv_features(const void* cells, void* feat, long long frames, int rows, int cols, int oh, int ow,
                                     int stride, int pad, int dil, void* stream) {
  const EmbConvGeom g{rows, cols, oh, ow, stride, pad, dil};
  if (!geom_ok(g) || frames < 0) return 1;
  if (reinterpret_cast<uintptr_t>(feat) % 16 != 0) return 2;
  const long long total = frames * (long long)(oh * ow);
  if (total == 0) return 0;
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffll) return 1;
  embconv_features_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int*>(cells), reinterpret_cast<elem_t*>(feat), frames, g);
  return launch_result();
}

// table: bf16 [vocab][9][O]; pos: fp32 [oh*ow][O] or null; z: bf16 [frames][oh*ow][O], read (when z_has_input) and
// overwritten with the pre-activation; y: bf16 like z or null, receives GELU(z) (or z itself without apply_gelu).
extern "C" int fbam_embconv_fwd(const void* cells, const void* table, const void* pos, void* z, void* y,
                                long long frames, int vocab, int O, int rows, int cols, int oh, int ow, int stride,
                                int pad, int dil, int seg_len, int z_has_input, int apply_gelu, void* stream) {
  const EmbConvGeom g{rows, cols, oh, ow, stride, pad, dil};
  if (!geom_ok(g) || frames < 0 || vocab < 1 || O < 8 || O % 8 != 0 || seg_len < 1) return 1;
  if (reinterpret_cast<uintptr_t>(table) % 16 != 0 || reinterpret_cast<uintptr_t>(z) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(y) % 16 != 0 || reinterpret_cast<uintptr_t>(pos) % 16 != 0)
    return 2;
  if (frames == 0) return 0;
  const int nseg = (int)((frames + seg_len - 1) / seg_len);
  const long long items = (long long)oh * ow * nseg;
  const long long blocks = (items + 7) / 8;
  if (blocks > 0x7fffffffll) return 1;
  dim3 grid((unsigned)blocks, (unsigned)((O + 255) / 256));
  embconv_fwd_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int*>(cells), reinterpret_cast<const elem_t*>(table), reinterpret_cast<const float*>(pos),
      reinterpret_cast<elem_t*>(z), reinterpret_cast<elem_t*>(y), frames, vocab, O, g, seg_len, nseg, z_has_input,
      apply_gelu);
  return launch_result();
}

// S: fp32 [vocab][9][O] and D: fp32 [oh*ow][O]; both are added to (the caller zeroes them).
extern "C" int fbam_embconv_bwd_reduce(const void* cells, const void* dz, void* S, void* D, long long frames, int vocab,
                                       int O, int rows, int cols, int oh, int ow, int stride, int pad, int dil,
                                       int seg_len, void* stream) {
  const EmbConvGeom g{rows, cols, oh, ow, stride, pad, dil};
  if (!geom_ok(g) || frames < 0 || vocab < 1 || O < 8 || O % 8 != 0 || seg_len < 1) return 1;
  if (reinterpret_cast<uintptr_t>(dz) % 16 != 0 || reinterpret_cast<uintptr_t>(S) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(D) % 16 != 0)
    return 2;
  if (frames == 0) return 0;
  const int nseg = (int)((frames + seg_len - 1) / seg_len);
  const long long items = (long long)oh * ow * nseg;
  const long long blocks = (items + 7) / 8;
  if (blocks > 0x7fffffffll) return 1;
  dim3 grid((unsigned)blocks, (unsigned)((O + 127) / 128));
  embconv_bwd_reduce_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int*>(cells), reinterpret_cast<const elem_t*>(dz), reinterpret_cast<float*>(S),
      reinterpret_cast<float*>(D), frames, vocab, O, g, seg_len, nseg);
  return launch_result();
}

// out[i] = sum over `slabs` fp32 slabs of n elements each (n a multiple of 4, 16-byte aligned pointers).
extern "C" int fbam_slab_reduce(const void* work, void* out, long long n, int slabs, int out_elem, void* stream) {
  if (n < 0 || n % 4 != 0 || slabs < 1) return 1;
  if (reinterpret_cast<uintptr_t>(work) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % (out_elem ? 8 : 16) != 0) return 2;
  if (n == 0) return 0;
  const long long blocks = (n / 4 + 255) / 256;
  slab_reduce_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float*>(work), out, n, slabs, out_elem);
  return launch_result();
}
