// Bandwidth-bound kernels (no tensor cores): normalisation, activations, pooling, cell embedding,
// cross-entropy, bias-gradient reductions and the fused optimizer update.  All are written for
// 16-byte vector accesses on bf16 data with fp32 arithmetic, one pass over memory per tensor, grids
// sized from the problem (rows or 16-byte packets), and predicated tails.
//
// Reference kernel families covered: build_cell_embeds and its three backward kernels
// (kernel_gen/kernel_gen/kernels/build_cell_embeds.py:23-248, build_cell_embeds_bwd.py:6-322), rms_norm fwd / bwd
// (kernels/rms_norm.py:14-104), layer_norm fwd (kernels/layer_norm.py:13-90; the backward here has no counterpart there), cross_entropy_on_targets fwd / bwd
// (kernels/cross_entropy.py:23-58, cross_entropy_bwd.py:22-66), avg_pool2d NHWC 2x2 fwd / bwd and the mean over
// positions (kernels/avg_pool2d.py:35-144, avg_pool2d_bwd.py:6-214, mean_reduce.py:30-108), column sums for bias
// gradients (kernels/sum_reduce.py:33-140), GELU / GeGLU and their gradients (kernels/act.py:43-86), and the AdamW
// and SGD steps (kernels/optimizer.py:6-79).
#include "elem16.cuh"
#include <cuda_runtime.h>
#include <stdint.h>

#include "gelu_math.cuh"

namespace {


__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `scratch` holds 32 floats.  Result is valid in every thread.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : 0.0f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    t = warp_max(t);
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

// GELU (exact erf form) and its derivative, eight values at a time on packed fp32 pairs (gelu_math.cuh)
__device__ __forceinline__ void gelu8(const float* x, float* y) {
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const float2 g = gelu_math::gelu2(make_float2(x[j], x[j + 1]));
    y[j] = g.x;
    y[j + 1] = g.y;
  }
}
__device__ __forceinline__ void gelu_grad8(const float* x, float* y) {
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const float2 g = gelu_math::gelu_grad2(make_float2(x[j], x[j + 1]));
    y[j] = g.x;
    y[j + 1] = g.y;
  }
}

struct alignas(16) Pack8 { elem2_t h[4]; };
__device__ __forceinline__ void unpack8(const Pack8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = e22ff(p.h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ Pack8 pack8(const float* f) {
  Pack8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.h[i] = ff2e2(f[2 * i], f[2 * i + 1]);
  return p;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm: one warp per row for dim <= 2048 (kept in registers), bf16 IO, fp32 math.
// ------------------------------------------------------------------------------------------------
template <int VEC_PER_LANE>  // dim = VEC_PER_LANE * 32 * 8 at most
__global__ void rmsnorm_fwd_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ w, elem_t* __restrict__ y,
                                   float* __restrict__ rstd, long long rows, int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const elem_t* xr = x + row * dim;
  float v[VEC_PER_LANE][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VEC_PER_LANE; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < dim) {
      unpack8(*reinterpret_cast<const Pack8*>(xr + c), v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / dim + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < VEC_PER_LANE; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < dim) {
      float g[8], o[8];
      unpack8(*reinterpret_cast<const Pack8*>(w + c), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * r * g[j];
      *reinterpret_cast<Pack8*>(y + row * dim + c) = pack8(o);
    }
  }
}

// dx = rstd * (g*dy - xhat * mean(g*dy*xhat));  dgamma[c] += sum_rows dy*xhat (fp32 atomics, one per
// column per block after an in-block reduction over the block's rows).
template <int VEC_PER_LANE>
__global__ void rmsnorm_bwd_kernel(const elem_t* __restrict__ dy, const elem_t* __restrict__ x, const elem_t* __restrict__ w,
                                   const float* __restrict__ rstd, elem_t* __restrict__ dx, float* __restrict__ dgamma,
                                   long long rows, int dim, int rows_per_warp) {
  extern __shared__ float sm_dg[];  // [dim]
  for (int c = threadIdx.x; c < dim; c += blockDim.x) sm_dg[c] = 0.0f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  float acc[VEC_PER_LANE][8];
#pragma unroll
  for (int i = 0; i < VEC_PER_LANE; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
  float g[VEC_PER_LANE][8];
#pragma unroll
  for (int i = 0; i < VEC_PER_LANE; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < dim) unpack8(*reinterpret_cast<const Pack8*>(w + c), g[i]);
  }
  const long long first = ((long long)blockIdx.x * warps + (threadIdx.x >> 5)) * rows_per_warp;
  for (int rr = 0; rr < rows_per_warp; ++rr) {
    const long long row = first + rr;
    if (row >= rows) break;
    const float r = rstd[row];
    float xv[VEC_PER_LANE][8], dv[VEC_PER_LANE][8];
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < dim) {
        unpack8(*reinterpret_cast<const Pack8*>(x + row * dim + c), xv[i]);
        unpack8(*reinterpret_cast<const Pack8*>(dy + row * dim + c), dv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xv[i][j] *= r;  // xhat
          acc[i][j] += dv[i][j] * xv[i][j];
          dot += dv[i][j] * g[i][j] * xv[i][j];
        }
      }
    }
    dot = warp_sum(dot) / dim;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < dim) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (dv[i][j] * g[i][j] - xv[i][j] * dot);
        *reinterpret_cast<Pack8*>(dx + row * dim + c) = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VEC_PER_LANE; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < dim)
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&sm_dg[c + j], acc[i][j]);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < dim; c += blockDim.x) atomicAdd(&dgamma[c], sm_dg[c]);
}

// LayerNorm forward (block per row).
__global__ void layernorm_fwd_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ w, const elem_t* __restrict__ b,
                                     elem_t* __restrict__ y, int dim, float eps) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const elem_t* xr = x + row * dim;
  float s = 0.0f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) s += e2f(xr[c]);
  const float mean = block_sum(s, scratch) / dim;
  float q = 0.0f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    const float d = e2f(xr[c]) - mean;
    q += d * d;
  }
  const float r = rsqrtf(block_sum(q, scratch) / dim + eps);
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float o = (e2f(xr[c]) - mean) * r * e2f(w[c]);
    if (b != nullptr) o += e2f(b[c]);
    y[row * dim + c] = f2e(o);
  }
}

// LayerNorm forward that also keeps the row statistics for the backward.
__global__ void layernorm_fwd_stats_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ w,
                                           const elem_t* __restrict__ b, elem_t* __restrict__ y, float* __restrict__ mean_out,
                                           float* __restrict__ rstd_out, int dim, float eps) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const elem_t* xr = x + row * dim;
  float s = 0.0f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) s += e2f(xr[c]);
  const float mean = block_sum(s, scratch) / dim;
  float q = 0.0f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    const float d = e2f(xr[c]) - mean;
    q += d * d;
  }
  const float r = rsqrtf(block_sum(q, scratch) / dim + eps);
  if (threadIdx.x == 0) {
    mean_out[row] = mean;
    rstd_out[row] = r;
  }
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float o = (e2f(xr[c]) - mean) * r * e2f(w[c]);
    if (b != nullptr) o += e2f(b[c]);
    y[row * dim + c] = f2e(o);
  }
}

// LayerNorm backward.  With xh = (x - mean) * rstd and g = dy * w:
//   dx = rstd * (g - mean_c(g) - xh * mean_c(g * xh)),   dw[c] += sum_rows dy * xh,   db[c] += sum_rows dy.
// A block walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; a thread owns columns threadIdx.x + k * blockDim.x
// (k < COLS) and keeps their dw / db sums in registers across its rows: one atomic per column and block at the end.
template <int COLS>
__global__ void __launch_bounds__(256) layernorm_bwd_kernel(const elem_t* __restrict__ dy, const elem_t* __restrict__ x,
                                                            const elem_t* __restrict__ w, const float* __restrict__ mean,
                                                            const float* __restrict__ rstd, elem_t* __restrict__ dx,
                                                            float* __restrict__ dw, float* __restrict__ db,
                                                            long long rows, int dim) {
  __shared__ float scratch[32];
  float wreg[COLS], dw_acc[COLS], db_acc[COLS];
#pragma unroll
  for (int k = 0; k < COLS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    wreg[k] = c < dim ? e2f(w[c]) : 0.0f;
    dw_acc[k] = 0.0f;
    db_acc[k] = 0.0f;
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float m = mean[row], r = rstd[row];
    float xh[COLS], g[COLS];
    float sg = 0.0f, sgx = 0.0f;
#pragma unroll
    for (int k = 0; k < COLS; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      xh[k] = 0.0f;
      g[k] = 0.0f;
      if (c < dim) {
        const float d = e2f(dy[row * dim + c]);
        xh[k] = (e2f(x[row * dim + c]) - m) * r;
        g[k] = d * wreg[k];
        dw_acc[k] += d * xh[k];
        db_acc[k] += d;
        sg += g[k];
        sgx += g[k] * xh[k];
      }
    }
    const float mg = block_sum(sg, scratch) / dim;
    const float mgx = block_sum(sgx, scratch) / dim;
#pragma unroll
    for (int k = 0; k < COLS; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      if (c < dim) dx[row * dim + c] = f2e(r * (g[k] - mg - xh[k] * mgx));
    }
  }
#pragma unroll
  for (int k = 0; k < COLS; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < dim) {
      atomicAdd(dw + c, dw_acc[k]);
      if (db != nullptr) atomicAdd(db + c, db_acc[k]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// element-wise
// ------------------------------------------------------------------------------------------------
// mode 0: y = gelu(x); mode 1: dx = dy * gelu'(x)
__global__ void gelu_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ dy, elem_t* __restrict__ out,
                            long long n8, int mode) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float a[8], o[8];
  unpack8(reinterpret_cast<const Pack8*>(x)[i], a);
  if (mode == 0) {
    gelu8(a, o);
  } else {
    float d[8];
    unpack8(reinterpret_cast<const Pack8*>(dy)[i], d);
    gelu_grad8(a, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] *= d[j];
  }
  reinterpret_cast<Pack8*>(out)[i] = pack8(o);
}

// GeGLU over the channel dimension: x [rows, 2C] -> y [rows, C] = value * gelu(gate).
__global__ void geglu_fwd_kernel(const elem_t* __restrict__ x, elem_t* __restrict__ y, long long rows, int c) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int c8 = c / 8;
  if (i >= rows * c8) return;
  const long long row = i / c8;
  const int col = (int)(i % c8) * 8;
  float v[8], g[8], o[8];
  unpack8(*reinterpret_cast<const Pack8*>(x + row * 2 * c + col), v);
  unpack8(*reinterpret_cast<const Pack8*>(x + row * 2 * c + c + col), g);
  gelu8(g, o);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] *= v[j];
  *reinterpret_cast<Pack8*>(y + row * c + col) = pack8(o);
}
__global__ void geglu_bwd_kernel(const elem_t* __restrict__ x, const elem_t* __restrict__ dy, elem_t* __restrict__ dx,
                                 long long rows, int c) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int c8 = c / 8;
  if (i >= rows * c8) return;
  const long long row = i / c8;
  const int col = (int)(i % c8) * 8;
  float v[8], g[8], d[8], dv[8], dg[8];
  unpack8(*reinterpret_cast<const Pack8*>(x + row * 2 * c + col), v);
  unpack8(*reinterpret_cast<const Pack8*>(x + row * 2 * c + c + col), g);
  unpack8(*reinterpret_cast<const Pack8*>(dy + row * c + col), d);
  gelu8(g, dv);
  gelu_grad8(g, dg);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    dv[j] *= d[j];
    dg[j] *= d[j] * v[j];
  }
  *reinterpret_cast<Pack8*>(dx + row * 2 * c + col) = pack8(dv);
  *reinterpret_cast<Pack8*>(dx + row * 2 * c + c + col) = pack8(dg);
}

// 2x2 stride-2 average pool, NHWC.  bwd=1 scatters dy/4 back.
__global__ void avgpool2x2_kernel(const elem_t* __restrict__ in, elem_t* __restrict__ out, long long n, int oh, int ow,
                                  int c, int bwd) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int c8 = c / 8;
  const long long total = n * oh * ow * c8;
  if (i >= total) return;
  const int col = (int)(i % c8) * 8;
  long long pix = i / c8;
  const int x = (int)(pix % ow);
  pix /= ow;
  const int y = (int)(pix % oh);
  const long long b = pix / oh;
  const int ih = oh * 2, iw = ow * 2;
  const long long obase = ((b * oh + y) * ow + x) * c + col;
  if (!bwd) {
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int dy = 0; dy < 2; ++dy)
#pragma unroll
      for (int dx = 0; dx < 2; ++dx) {
        float v[8];
        unpack8(*reinterpret_cast<const Pack8*>(in + ((b * ih + 2 * y + dy) * iw + 2 * x + dx) * c + col), v);
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] += v[j];
      }
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] *= 0.25f;
    *reinterpret_cast<Pack8*>(out + obase) = pack8(s);
  } else {
    float v[8];
    unpack8(*reinterpret_cast<const Pack8*>(in + obase), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= 0.25f;
    const Pack8 p = pack8(v);
#pragma unroll
    for (int dy = 0; dy < 2; ++dy)
#pragma unroll
      for (int dx = 0; dx < 2; ++dx)
        *reinterpret_cast<Pack8*>(out + ((b * ih + 2 * y + dy) * iw + 2 * x + dx) * c + col) = p;
  }
}

// Global average pool over `pix` positions: x [n, pix, c] -> y [n, c].  One block per (n, 8-channel-group
// slab of 32 groups); threads stride over positions.
__global__ void global_avgpool_fwd_kernel(const elem_t* __restrict__ x, elem_t* __restrict__ y, int pix, int c) {
  __shared__ float red[8][33][8];
  const long long n = blockIdx.x;
  const int cg = blockIdx.y * 32 + (threadIdx.x & 31);  // 8-channel group
  const int slice = threadIdx.x >> 5;                   // 8 slices over positions
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cg * 8 < c) {
    for (int p = slice; p < pix; p += 8) {
      float v[8];
      unpack8(*reinterpret_cast<const Pack8*>(x + (n * pix + p) * c + cg * 8), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[slice][threadIdx.x & 31][j] = s[j];
  __syncthreads();
  if (slice == 0 && cg * 8 < c) {
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x & 31][j];
      o[j] = t / pix;
    }
    *reinterpret_cast<Pack8*>(y + n * c + cg * 8) = pack8(o);
  }
}
// dx[n, p, :] = dy[n, :] / pix, optionally multiplied by gelu'(z[n, p, :]) (z = pre-activation of the
// GELU that fed the pool), which folds the activation gradient into the same pass.  Grid-stride over 16-byte
// groups, four per thread and trip with all loads issued before the arithmetic; I is a 32-bit index type whenever
// the group count fits one (64-bit division costs more than the rest of the thread's work).
template <typename I>
__global__ void __launch_bounds__(256) global_avgpool_bwd_kernel(const elem_t* __restrict__ dy, const elem_t* __restrict__ z,
                                                                 elem_t* __restrict__ dx, I total, I pix, I c8) {
  constexpr int kUnroll = 4;
  const I stride = (I)gridDim.x * blockDim.x;
  const I per_image = pix * c8;
  const float inv = 1.0f / (float)pix;
  for (I base = (I)blockIdx.x * blockDim.x + threadIdx.x; base < total; base += stride * kUnroll) {
    Pack8 zr[kUnroll], dr[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const I i = base + (I)u * stride;
      if (i < total) {
        if (z != nullptr) zr[u] = reinterpret_cast<const Pack8*>(z)[i];
        dr[u] = reinterpret_cast<const Pack8*>(dy)[(i / per_image) * c8 + i % c8];
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const I i = base + (I)u * stride;
      if (i >= total) continue;
      float v[8];
      unpack8(dr[u], v);
      if (z != nullptr) {
        float zv[8], gz[8];
        unpack8(zr[u], zv);
        gelu_grad8(zv, gz);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= inv * gz[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= inv;
      }
      reinterpret_cast<Pack8*>(dx)[i] = pack8(v);
    }
  }
}

// Column sums of a bf16 matrix [rows, cols] into fp32 (bias gradients): out[c] += sum_r x[r, c].
__global__ void colsum_kernel(const elem_t* __restrict__ x, float* __restrict__ out, long long rows, int cols,
                              int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= cols) return;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(rows, r0 + rows_per_block);
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (long long r = r0; r < r1; ++r) {
    float v[8];
    unpack8(*reinterpret_cast<const Pack8*>(x + r * cols + c), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] += v[j];
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) atomicAdd(out + c + j, s[j]);
}

// ------------------------------------------------------------------------------------------------
// cell embedding
// ------------------------------------------------------------------------------------------------
// out[f, p, :] = cp_embed[cp] (0 if out of range) + pos_embed[p] + sum_c chan_c/255 * colour[c]
// A thread owns (position p, 8 channels) and walks a slice of the frames: its position row and the six
// colour vectors stay in registers, so per cell it loads only the three cell words and one slice of the
// code-point table and stores 16 bytes.  The threads of a block cover 16 neighbouring positions x all channels,
// i.e. one contiguous 4 KB span of the output per frame.  When the code-point table fits (SMEM_TABLE), a bf16
// copy of it is staged in shared memory once per block (rows padded by 16 bytes against bank conflicts), which
// removes the table's L2 traffic — otherwise 2 bytes read per byte written.
template <bool SMEM_TABLE>
__global__ void __launch_bounds__(512) cell_embed_fwd_kernel(const int* __restrict__ cells, const float* __restrict__ cp_embed,
                                      const float* __restrict__ pos_embed, const float* __restrict__ colour,
                                      elem_t* __restrict__ out, long long frames, int positions, int e, int vocab,
                                      int frames_per_block) {
  extern __shared__ uint4 embed_smem[];
  const int e8 = e / 8;
  const int row_u4 = e8 + 1;   // padded row length in 16-byte units
  if (SMEM_TABLE) {
    for (int i = threadIdx.x; i < vocab * e8; i += blockDim.x) {
      const int r = i / e8, c = i % e8;
      const float4* src = reinterpret_cast<const float4*>(cp_embed + (long long)r * e + c * 8);
      const float4 a = src[0], b = src[1];
      const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      const Pack8 pk = pack8(f);
      embed_smem[r * row_u4 + c] = *reinterpret_cast<const uint4*>(&pk);
    }
    __syncthreads();
  }
  const int g = threadIdx.x % e8, pl = threadIdx.x / e8;
  const int p = blockIdx.x * (blockDim.x / e8) + pl;
  if (p >= positions) return;
  const int col = g * 8;
  float pos[8], cv[6][8];
  {
    const float4* pe = reinterpret_cast<const float4*>(pos_embed + (long long)p * e + col);
    const float4 a = pe[0], b = pe[1];
    pos[0] = a.x; pos[1] = a.y; pos[2] = a.z; pos[3] = a.w; pos[4] = b.x; pos[5] = b.y; pos[6] = b.z; pos[7] = b.w;
#pragma unroll
    for (int k = 0; k < 6; ++k) {
      const float4* c4 = reinterpret_cast<const float4*>(colour + k * e + col);
      const float4 x = c4[0], y = c4[1];
      cv[k][0] = x.x; cv[k][1] = x.y; cv[k][2] = x.z; cv[k][3] = x.w;
      cv[k][4] = y.x; cv[k][5] = y.y; cv[k][6] = y.z; cv[k][7] = y.w;
    }
  }
  const long long f0 = (long long)blockIdx.y * frames_per_block;
  const long long f1 = min(frames, f0 + frames_per_block);
  constexpr int G = 8;   // frames whose cell words are fetched together (loads in flight per thread)
  for (long long fb = f0; fb < f1; fb += G) {
    int cpq[G];
    uint32_t fgq[G], bgq[G];
#pragma unroll
    for (int u = 0; u < G; ++u) {
      const long long f = fb + u;
      if (f < f1) {
        const int* cw = cells + (f * positions + p) * 3;
        cpq[u] = cw[0];
        fgq[u] = (uint32_t)cw[1];
        bgq[u] = (uint32_t)cw[2];
      }
    }
#pragma unroll
    for (int u = 0; u < G; ++u) {
      const long long f = fb + u;
      if (f >= f1) break;
      const long long cell = f * positions + p;
      const int cp = cpq[u];
      const uint32_t fg = fgq[u], bg = bgq[u];
      const float ch[6] = {((fg >> 16) & 255) * (1.0f / 255.0f), ((fg >> 8) & 255) * (1.0f / 255.0f),
                           (fg & 255) * (1.0f / 255.0f),         ((bg >> 16) & 255) * (1.0f / 255.0f),
                           ((bg >> 8) & 255) * (1.0f / 255.0f),  (bg & 255) * (1.0f / 255.0f)};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = pos[j];
      if (cp >= 0 && cp < vocab) {
        if (SMEM_TABLE) {
          float t[8];
          const uint4 raw = embed_smem[cp * row_u4 + g];
          unpack8(*reinterpret_cast<const Pack8*>(&raw), t);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += t[j];
        } else {
          const float4* ce = reinterpret_cast<const float4*>(cp_embed + (long long)cp * e + col);
          const float4 a = ce[0], b = ce[1];
          o[0] += a.x; o[1] += a.y; o[2] += a.z; o[3] += a.w; o[4] += b.x; o[5] += b.y; o[6] += b.z; o[7] += b.w;
        }
      }
#pragma unroll
      for (int k = 0; k < 6; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += ch[k] * cv[k][j];
      *reinterpret_cast<Pack8*>(out + cell * e + col) = pack8(o);
    }
  }
}

// Backward of the cell embedding, all three tables in one pass over dOut.  A thread owns (position p,
// 8 channels) and walks a slice of the frames:
//   * position gradient: running sum, one atomic per slice;
//   * colour gradients: running weighted sums, reduced over the block in shared memory, then one atomic
//     per (colour, channel) per block;
//   * code-point gradient: consecutive frames mostly show the same glyph at a position, so the thread
//     accumulates while the code point stays the same and issues its 8 atomics only when it changes
//     (run-length flushing); worst case (every frame differs) this degenerates to one flush per cell.
__global__ void cell_embed_bwd_kernel(const int* __restrict__ cells, const elem_t* __restrict__ dout,
                                      float* __restrict__ d_cp, float* __restrict__ d_pos,
                                      float* __restrict__ d_colour, long long frames, int positions, int e, int vocab,
                                      int frames_per_block) {
  extern __shared__ float sm_col[];  // [6][e]
  for (int i = threadIdx.x; i < 6 * e; i += blockDim.x) sm_col[i] = 0.0f;
  __syncthreads();
  const int e8 = e / 8;
  const int g = threadIdx.x % e8, pl = threadIdx.x / e8;
  const int p = blockIdx.x * (blockDim.x / e8) + pl;
  const long long f0 = (long long)blockIdx.y * frames_per_block;
  const long long f1 = min(frames, f0 + frames_per_block);
  const int col = g * 8;
  if (p < positions) {
    float pos_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float run_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int run_cp = -1;
    float col_acc[6][8];
#pragma unroll
    for (int k = 0; k < 6; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) col_acc[k][j] = 0.0f;
    for (long long fb = f0; fb < f1; fb += 4) {
     // issue the loads of four frames before touching any of them (memory-level parallelism)
     Pack8 dq[4];
     int cpq[4];
     uint32_t fgq[4], bgq[4];
#pragma unroll
     for (int u = 0; u < 4; ++u) {
       const long long f = fb + u;
       if (f < f1) {
         const long long cell = f * positions + p;
         dq[u] = *reinterpret_cast<const Pack8*>(dout + cell * e + col);
         cpq[u] = cells[cell * 3 + 0];
         fgq[u] = (uint32_t)cells[cell * 3 + 1];
         bgq[u] = (uint32_t)cells[cell * 3 + 2];
       }
     }
#pragma unroll
     for (int u = 0; u < 4; ++u) {
      if (fb + u >= f1) break;
      float d[8];
      unpack8(dq[u], d);
      const int cp = cpq[u];
      const uint32_t fg = fgq[u], bg = bgq[u];
      const float ch[6] = {((fg >> 16) & 255) * (1.0f / 255.0f), ((fg >> 8) & 255) * (1.0f / 255.0f),
                           (fg & 255) * (1.0f / 255.0f),         ((bg >> 16) & 255) * (1.0f / 255.0f),
                           ((bg >> 8) & 255) * (1.0f / 255.0f),  (bg & 255) * (1.0f / 255.0f)};
      if (cp != run_cp) {
        if (run_cp >= 0 && run_cp < vocab) {
          float* dst = d_cp + (long long)run_cp * e + col;
#pragma unroll
          for (int j = 0; j < 8; ++j) atomicAdd(dst + j, run_acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) run_acc[j] = 0.0f;
        run_cp = cp;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        pos_acc[j] += d[j];
        run_acc[j] += d[j];
      }
#pragma unroll
      for (int k = 0; k < 6; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) col_acc[k][j] += ch[k] * d[j];
     }
    }
    if (run_cp >= 0 && run_cp < vocab) {
      float* dst = d_cp + (long long)run_cp * e + col;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, run_acc[j]);
    }
    float* dp = d_pos + (long long)p * e + col;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dp + j, pos_acc[j]);
#pragma unroll
    for (int k = 0; k < 6; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&sm_col[k * e + col + j], col_acc[k][j]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 6 * e; i += blockDim.x) atomicAdd(d_colour + i, sm_col[i]);
}

// ------------------------------------------------------------------------------------------------
// cross-entropy on bf16 logits, forward + backward in one pass over the row
// ------------------------------------------------------------------------------------------------
// logits [rows, ld] (first `vocab` columns valid).  loss_sum += scale * sum_rows (lse - logit[target]);
// logits are overwritten with scale * (softmax - onehot); padding columns get 0.
__global__ void ce_fwd_bwd_kernel(elem_t* __restrict__ logits, const long long* __restrict__ targets,
                                  float* __restrict__ loss_sum, int vocab, int ld, float scale, int write_grad) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  elem_t* lr = logits + row * ld;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) mx = fmaxf(mx, e2f(lr[c]));
  mx = block_max(mx, scratch);
  float s = 0.0f;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) s += __expf(e2f(lr[c]) - mx);
  s = block_sum(s, scratch);
  const int t = (int)targets[row];
  if (threadIdx.x == 0) {
    const float lt = (t >= 0 && t < vocab) ? e2f(lr[t]) : 0.0f;
    atomicAdd(loss_sum, scale * (logf(s) + mx - lt));
  }
  if (!write_grad) return;
  const float inv = 1.0f / s;
  for (int c = threadIdx.x; c < ld; c += blockDim.x) {
    float g = 0.0f;
    if (c < vocab) g = scale * (__expf(e2f(lr[c]) - mx) * inv - (c == t ? 1.0f : 0.0f));
    lr[c] = f2e(g);
  }
}

// Fused LM head + cross-entropy, second step: the head GEMM's epilogue left, per row and tile half, the maximum of
// the logits and the sum of exp relative to it (and the target logit); one thread per row merges them into the
// row's log-sum-exp and adds scale * (lse - target logit) to the loss.
__global__ void ce_combine_kernel(const float* __restrict__ partial, const float* __restrict__ tgt_logit,
                                  float* __restrict__ lse, float* __restrict__ loss_sum, long long rows, int slots,
                                  float scale) {
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float contrib = 0.0f;
  if (row < rows) {
    const float* pr = partial + row * slots * 2;
    float m = -INFINITY;
    for (int s = 0; s < slots; ++s) m = fmaxf(m, pr[2 * s]);
    float sum = 0.0f;
    for (int s = 0; s < slots; ++s)
      if (pr[2 * s] > -INFINITY) sum += pr[2 * s + 1] * __expf(pr[2 * s] - m);
    const float l = m + logf(sum);
    lse[row] = l;
    contrib = scale * (l - tgt_logit[row]);
  }
  contrib = warp_sum(contrib);
  if ((threadIdx.x & 31) == 0 && contrib != 0.0f) atomicAdd(loss_sum, contrib);
}

// Same with fp32 logits in (the LM-head GEMM keeps its fp32 accumulators) and bf16 gradient out: the loss and the
// softmax are then free of the bf16 rounding of the logits.
__global__ void ce_fwd_bwd_f32_kernel(const float* __restrict__ logits, elem_t* __restrict__ dlogits,
                                      const long long* __restrict__ targets, float* __restrict__ loss_sum, int vocab,
                                      int ld, float scale) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const float* lr = logits + row * ld;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) mx = fmaxf(mx, lr[c]);
  mx = block_max(mx, scratch);
  float s = 0.0f;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) s += __expf(lr[c] - mx);
  s = block_sum(s, scratch);
  const int t = (int)targets[row];
  if (threadIdx.x == 0) {
    const float lt = (t >= 0 && t < vocab) ? lr[t] : 0.0f;
    atomicAdd(loss_sum, scale * (logf(s) + mx - lt));
  }
  if (dlogits == nullptr) return;
  const float inv = 1.0f / s;
  elem_t* dr = dlogits + row * ld;
  for (int c = threadIdx.x; c < ld; c += blockDim.x) {
    float g = 0.0f;
    if (c < vocab) g = scale * (__expf(lr[c] - mx) * inv - (c == t ? 1.0f : 0.0f));
    dr[c] = f2e(g);
  }
}

// ------------------------------------------------------------------------------------------------
// fused AdamW over a flat range: reads g (bf16 or fp32), updates m, v, fp32 master and writes the
// rounded parameter.  4 elements per thread.
// ------------------------------------------------------------------------------------------------
template <typename PT>
__global__ void adamw_kernel(PT* __restrict__ param, const PT* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, float* __restrict__ master, long long n, float lr, float b1,
                             float b2, float eps, float wd, float inv_bc1, float inv_bc2, float grad_scale, int vec_ok) {
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i0 >= n) return;
  const bool vec = vec_ok && i0 + 4 <= n;   // 16-byte accesses when the launcher found every pointer aligned
  float g[4], w[4], mm[4], vv[4];
  if (vec) {
    const float4 tm = *reinterpret_cast<const float4*>(m + i0), tv = *reinterpret_cast<const float4*>(v + i0);
    mm[0] = tm.x; mm[1] = tm.y; mm[2] = tm.z; mm[3] = tm.w;
    vv[0] = tv.x; vv[1] = tv.y; vv[2] = tv.z; vv[3] = tv.w;
    if constexpr (sizeof(PT) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(grad + i0);
      const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
      const float2 a = e22ff(h[0]), b = e22ff(h[1]);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      const float4 tg = *reinterpret_cast<const float4*>(grad + i0);
      g[0] = tg.x; g[1] = tg.y; g[2] = tg.z; g[3] = tg.w;
    }
    if (master != nullptr) {
      const float4 tw = *reinterpret_cast<const float4*>(master + i0);
      w[0] = tw.x; w[1] = tw.y; w[2] = tw.z; w[3] = tw.w;
    } else if constexpr (sizeof(PT) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(param + i0);
      const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
      const float2 a = e22ff(h[0]), b = e22ff(h[1]);
      w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
    } else {
      const float4 tw = *reinterpret_cast<const float4*>(param + i0);
      w[0] = tw.x; w[1] = tw.y; w[2] = tw.z; w[3] = tw.w;
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const long long i = i0 + k;
    if (!vec) {
      if (i >= n) return;
      if constexpr (sizeof(PT) == 2) g[k] = e2f(grad[i]); else g[k] = grad[i];
      if (master != nullptr) w[k] = master[i];
      else if constexpr (sizeof(PT) == 2) w[k] = e2f(param[i]); else w[k] = param[i];
      mm[k] = m[i];
      vv[k] = v[i];
    }
    const float gk = g[k] * grad_scale;
    w[k] *= 1.0f - lr * wd;
    mm[k] = b1 * mm[k] + (1.0f - b1) * gk;
    vv[k] = b2 * vv[k] + (1.0f - b2) * gk * gk;
    w[k] -= lr * (mm[k] * inv_bc1) / (sqrtf(vv[k] * inv_bc2) + eps);
    if (!vec) {
      m[i] = mm[k];
      v[i] = vv[k];
      if (master != nullptr) master[i] = w[k];
      if constexpr (sizeof(PT) == 2) param[i] = f2e(w[k]); else param[i] = w[k];
    }
  }
  if (vec) {
    *reinterpret_cast<float4*>(m + i0) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + i0) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (master != nullptr) *reinterpret_cast<float4*>(master + i0) = make_float4(w[0], w[1], w[2], w[3]);
    if constexpr (sizeof(PT) == 2) {
      __align__(8) elem2_t h[2] = {ff2e2(w[0], w[1]), ff2e2(w[2], w[3])};
      *reinterpret_cast<uint2*>(param + i0) = *reinterpret_cast<uint2*>(h);
    } else {
      *reinterpret_cast<float4*>(param + i0) = make_float4(w[0], w[1], w[2], w[3]);
    }
  }
}

template <int V>
int launch_rms_fwd(const elem_t* x, const elem_t* w, elem_t* y, float* rstd, long long rows, int dim, float eps,
                   cudaStream_t s) {
  const int warps = 8;
  rmsnorm_fwd_kernel<V><<<(unsigned)((rows + warps - 1) / warps), warps * 32, 0, s>>>(x, w, y, rstd, rows, dim, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}
template <int V>
int launch_rms_bwd(const elem_t* dy, const elem_t* x, const elem_t* w, const float* rstd, elem_t* dx, float* dg, long long rows,
                   int dim, cudaStream_t s) {
  const int warps = 8, rpw = 8;
  const long long blocks = (rows + warps * rpw - 1) / (warps * rpw);
  rmsnorm_bwd_kernel<V><<<(unsigned)blocks, warps * 32, dim * sizeof(float), s>>>(dy, x, w, rstd, dx, dg, rows, dim, rpw);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}


// -------------------------------------------------------------------------------------------------
// SGD step: g' = g + wd·w;  v = mu·v + g';  step = nesterov ? g' + mu·v : v  (no momentum: step = g');
// w -= lr·step.  w is the fp32 master copy when there is one, else the parameter itself.
// -------------------------------------------------------------------------------------------------
template <typename PT>
__global__ void sgd_kernel(PT* __restrict__ param, const PT* __restrict__ grad, float* __restrict__ velocity,
                           float* __restrict__ master, long long n, float lr, float mu, int nesterov, float wd) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float g, w;
  if constexpr (sizeof(PT) == 2) g = e2f(grad[i]); else g = grad[i];
  if (master != nullptr) w = master[i];
  else if constexpr (sizeof(PT) == 2) w = e2f(param[i]); else w = param[i];
  g += wd * w;
  if (velocity != nullptr) {
    const float v = mu * velocity[i] + g;
    velocity[i] = v;
    g = nesterov ? g + mu * v : v;
  }
  w -= lr * g;
  if (master != nullptr) master[i] = w;
  if constexpr (sizeof(PT) == 2) param[i] = f2e(w); else param[i] = w;
}

// -------------------------------------------------------------------------------------------------
// 128-bit content fingerprint of a buffer (shared-state comparison between peers): the sum, over all 8-byte
// words, of two independent 64-bit mixes of (word, index).  Sums commute, so the result does not depend on how
// the words are spread over threads.  A fingerprint for equality checks between cooperating peers, not a
// cryptographic hash.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__global__ void fingerprint_kernel(const unsigned long long* __restrict__ words, long long n_words,
                                   const unsigned char* __restrict__ tail, int tail_bytes,
                                   unsigned long long* __restrict__ out) {
  unsigned long long h0 = 0, h1 = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
    const unsigned long long w = words[i];
    const unsigned long long a = mix64(w + (unsigned long long)(i + 1) * 0x9E3779B97F4A7C15ull);
    h0 += a;
    h1 += mix64((a ^ 0xD6E8FEB86659FD93ull) + w);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && tail_bytes > 0) {
    unsigned long long w = 0;
    for (int b = 0; b < tail_bytes; ++b) w |= (unsigned long long)tail[b] << (8 * b);
    const unsigned long long a = mix64(w + (unsigned long long)(n_words + 1) * 0x9E3779B97F4A7C15ull);
    h0 += a;
    h1 += mix64((a ^ 0xD6E8FEB86659FD93ull) + w + (unsigned long long)tail_bytes);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    h0 += __shfl_xor_sync(0xffffffffu, h0, o);
    h1 += __shfl_xor_sync(0xffffffffu, h1, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(out, h0);
    atomicAdd(out + 1, h1);
  }
}

}  // namespace

#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : 5)

extern "C" {

int fbam_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int dim, float eps,
                     void* stream) {
  if (dim % 8 != 0 || dim > 8192) return 1;
  const elem_t *X = (const elem_t*)x, *W = (const elem_t*)w;
  if (dim <= 256) return launch_rms_fwd<1>(X, W, (elem_t*)y, rstd, rows, dim, eps, STREAM(stream));
  if (dim <= 512) return launch_rms_fwd<2>(X, W, (elem_t*)y, rstd, rows, dim, eps, STREAM(stream));
  if (dim <= 1024) return launch_rms_fwd<4>(X, W, (elem_t*)y, rstd, rows, dim, eps, STREAM(stream));
  if (dim <= 2048) return launch_rms_fwd<8>(X, W, (elem_t*)y, rstd, rows, dim, eps, STREAM(stream));
  if (dim <= 4096) return launch_rms_fwd<16>(X, W, (elem_t*)y, rstd, rows, dim, eps, STREAM(stream));
  return launch_rms_fwd<32>(X, W, (elem_t*)y, rstd, rows, dim, eps, STREAM(stream));
}

int fbam_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dgamma,
                     long long rows, int dim, void* stream) {
  if (dim % 8 != 0 || dim > 4096) return 1;
  const elem_t *DY = (const elem_t*)dy, *X = (const elem_t*)x, *W = (const elem_t*)w;
  if (dim <= 256) return launch_rms_bwd<1>(DY, X, W, rstd, (elem_t*)dx, dgamma, rows, dim, STREAM(stream));
  if (dim <= 512) return launch_rms_bwd<2>(DY, X, W, rstd, (elem_t*)dx, dgamma, rows, dim, STREAM(stream));
  if (dim <= 1024) return launch_rms_bwd<4>(DY, X, W, rstd, (elem_t*)dx, dgamma, rows, dim, STREAM(stream));
  if (dim <= 2048) return launch_rms_bwd<8>(DY, X, W, rstd, (elem_t*)dx, dgamma, rows, dim, STREAM(stream));
  return launch_rms_bwd<16>(DY, X, W, rstd, (elem_t*)dx, dgamma, rows, dim, STREAM(stream));
}

// partial: fp32 [rows][slots][2] (maximum, sum of exp) from the head GEMM's statistics epilogue; tgt_logit: fp32 [rows];
// lse: fp32 [rows] out; loss_sum: fp32 [1], added to.
int fbam_ce_combine(const float* partial, const float* tgt_logit, float* lse, float* loss_sum, long long rows, int slots,
                    float scale, void* stream) {
  if (rows < 0 || slots < 1) return 1;
  if (rows == 0) return 0;
  ce_combine_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, STREAM(stream)>>>(partial, tgt_logit, lse, loss_sum, rows,
                                                                               slots, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

// mean / rstd: fp32 [rows], kept for fbam_layernorm_bwd
int fbam_layernorm_fwd_stats(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                             long long rows, int dim, float eps, void* stream) {
  if (rows <= 0 || dim <= 0) return rows == 0 ? 0 : 1;
  layernorm_fwd_stats_kernel<<<(unsigned)rows, 256, 0, STREAM(stream)>>>((const elem_t*)x, (const elem_t*)w, (const elem_t*)b,
                                                                        (elem_t*)y, mean, rstd, dim, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

// dw, db: fp32 [dim], added to (the caller zeroes them); db may be null.  dim <= 8192.
int fbam_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                       float* dw, float* db, long long rows, int dim, void* stream) {
  if (rows <= 0 || dim <= 0) return rows == 0 ? 0 : 1;
  if (dim > 8192) return 1;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned grid = (unsigned)(rows < 4ll * sms ? rows : 4ll * sms);
  const elem_t *dyp = (const elem_t*)dy, *xp = (const elem_t*)x, *wp = (const elem_t*)w;
  cudaStream_t s = STREAM(stream);
  if (dim <= 1024) layernorm_bwd_kernel<4><<<grid, 256, 0, s>>>(dyp, xp, wp, mean, rstd, (elem_t*)dx, dw, db, rows, dim);
  else if (dim <= 2048) layernorm_bwd_kernel<8><<<grid, 256, 0, s>>>(dyp, xp, wp, mean, rstd, (elem_t*)dx, dw, db, rows, dim);
  else if (dim <= 4096) layernorm_bwd_kernel<16><<<grid, 256, 0, s>>>(dyp, xp, wp, mean, rstd, (elem_t*)dx, dw, db, rows, dim);
  else layernorm_bwd_kernel<32><<<grid, 256, 0, s>>>(dyp, xp, wp, mean, rstd, (elem_t*)dx, dw, db, rows, dim);
  return cudaGetLastError() == cudaSuccess ? 0 : 5;
}

int fbam_layernorm_fwd(const void* x, const void* w, const void* b, void* y, long long rows, int dim, float eps,
                       void* stream) {
  layernorm_fwd_kernel<<<(unsigned)rows, 256, 0, STREAM(stream)>>>((const elem_t*)x, (const elem_t*)w, (const elem_t*)b,
                                                                   (elem_t*)y, dim, eps);
  return CHECK_LAUNCH();
}

int fbam_gelu(const void* x, const void* dy, void* out, long long n, int mode, void* stream) {
  if (n % 8 != 0) return 1;
  const long long n8 = n / 8;
  gelu_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, STREAM(stream)>>>((const elem_t*)x, (const elem_t*)dy, (elem_t*)out,
                                                                        n8, mode);
  return CHECK_LAUNCH();
}

int fbam_geglu(const void* x, const void* dy, void* out, long long rows, int c, int bwd, void* stream) {
  if (c % 8 != 0) return 1;
  const long long n = rows * (c / 8);
  if (!bwd) geglu_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, STREAM(stream)>>>((const elem_t*)x, (elem_t*)out, rows, c);
  else geglu_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, STREAM(stream)>>>((const elem_t*)x, (const elem_t*)dy,
                                                                                (elem_t*)out, rows, c);
  return CHECK_LAUNCH();
}

int fbam_avgpool2x2(const void* in, void* out, long long n, int oh, int ow, int c, int bwd, void* stream) {
  if (c % 8 != 0) return 1;
  const long long total = n * oh * ow * (c / 8);
  avgpool2x2_kernel<<<(unsigned)((total + 255) / 256), 256, 0, STREAM(stream)>>>((const elem_t*)in, (elem_t*)out, n, oh, ow,
                                                                                 c, bwd);
  return CHECK_LAUNCH();
}

int fbam_global_avgpool(const void* in, void* out, long long n, int pix, int c, int bwd, const void* gelu_z,
                        void* stream) {
  if (c % 8 != 0) return 1;
  if (!bwd) {
    dim3 grid((unsigned)n, (c / 8 + 31) / 32);
    global_avgpool_fwd_kernel<<<grid, 256, 0, STREAM(stream)>>>((const elem_t*)in, (elem_t*)out, pix, c);
  } else {
    const long long total = n * pix * (c / 8);
    const long long want = (total + 256 * 4 - 1) / (256 * 4);
    const unsigned blocks = (unsigned)(want < 148 * 8 ? (want > 0 ? want : 1) : 148 * 8);
    if (total + 4LL * blocks * 256 < (1LL << 32))
      global_avgpool_bwd_kernel<unsigned><<<blocks, 256, 0, STREAM(stream)>>>(
          (const elem_t*)in, (const elem_t*)gelu_z, (elem_t*)out, (unsigned)total, (unsigned)pix, (unsigned)(c / 8));
    else
      global_avgpool_bwd_kernel<long long><<<blocks, 256, 0, STREAM(stream)>>>(
          (const elem_t*)in, (const elem_t*)gelu_z, (elem_t*)out, total, (long long)pix, (long long)(c / 8));
  }
  return CHECK_LAUNCH();
}

int fbam_colsum(const void* x, float* out, long long rows, int cols, void* stream) {
  if (cols % 8 != 0) return 1;
  const int threads = 128;
  const int gx = (cols / 8 + threads - 1) / threads;
  // rows per block: enough blocks to occupy every SM several times over (the loads of a thread are its only
  // memory parallelism), but at least 32 rows per block so that the atomics stay a small part of the work
  const long long want_gy = (148 * 8 + gx - 1) / gx;
  long long rpb = (rows + want_gy - 1) / want_gy;
  rpb = rpb < 32 ? 32 : (rpb > 256 ? 256 : rpb);
  dim3 grid(gx, (unsigned)((rows + rpb - 1) / rpb));
  colsum_kernel<<<grid, threads, 0, STREAM(stream)>>>((const elem_t*)x, out, rows, cols, (int)rpb);
  return CHECK_LAUNCH();
}

static int embed_threads(int e8) { return (256 / e8 > 0 ? 256 / e8 : 1) * e8; }

int fbam_cell_embed_fwd(const int* cells, const float* cp_embed, const float* pos_embed, const float* colour,
                        void* out, long long frames, int positions, int e, int vocab, void* stream) {
  if (e % 8 != 0 || e / 8 > 256) return 1;
  const int e8 = e / 8, threads = embed_threads(e8), ppb = threads / e8;
  const size_t table = (size_t)vocab * (e8 + 1) * 16;
  if (table <= 160 * 1024 && frames >= 256) {
    // code-point table staged in shared memory: larger frame slices amortise the staging
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(cell_embed_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) !=
          cudaSuccess)
        return 5;
      configured = true;
    }
    const int fpb = 256;
    const int big = (512 / e8 > 0 ? 512 / e8 : 1) * e8;   // one 512-thread block per SM next to the 136 KB table
    const int ppb2 = big / e8;
    dim3 grid((positions + ppb2 - 1) / ppb2, (unsigned)((frames + fpb - 1) / fpb));
    cell_embed_fwd_kernel<true><<<grid, big, table, STREAM(stream)>>>(cells, cp_embed, pos_embed, colour, (elem_t*)out,
                                                                      frames, positions, e, vocab, fpb);
    return CHECK_LAUNCH();
  }
  const int fpb = 64;
  dim3 grid((positions + ppb - 1) / ppb, (unsigned)((frames + fpb - 1) / fpb));
  cell_embed_fwd_kernel<false><<<grid, threads, 0, STREAM(stream)>>>(cells, cp_embed, pos_embed, colour, (elem_t*)out,
                                                                     frames, positions, e, vocab, fpb);
  return CHECK_LAUNCH();
}

int fbam_cell_embed_bwd(const int* cells, const void* dout, float* d_cp, float* d_pos, float* d_colour,
                        long long frames, int positions, int e, int vocab, void* stream) {
  if (e % 8 != 0 || e / 8 > 256) return 1;
  const int e8 = e / 8, threads = embed_threads(e8), ppb = threads / e8;
  const int fpb = 256;
  dim3 grid((positions + ppb - 1) / ppb, (unsigned)((frames + fpb - 1) / fpb));
  cell_embed_bwd_kernel<<<grid, threads, 6 * e * sizeof(float), STREAM(stream)>>>(
      cells, (const elem_t*)dout, d_cp, d_pos, d_colour, frames, positions, e, vocab, fpb);
  return CHECK_LAUNCH();
}

int fbam_ce_fwd_bwd(void* logits, const long long* targets, float* loss_sum, long long rows, int vocab, int ld,
                    float scale, int write_grad, void* stream) {
  ce_fwd_bwd_kernel<<<(unsigned)rows, 256, 0, STREAM(stream)>>>((elem_t*)logits, targets, loss_sum, vocab, ld, scale,
                                                                write_grad);
  return CHECK_LAUNCH();
}

int fbam_ce_fwd_bwd_f32(const float* logits, void* dlogits, const long long* targets, float* loss_sum, long long rows,
                        int vocab, int ld, float scale, void* stream) {
  ce_fwd_bwd_f32_kernel<<<(unsigned)rows, 256, 0, STREAM(stream)>>>(logits, (elem_t*)dlogits, targets, loss_sum, vocab, ld,
                                                                    scale);
  return CHECK_LAUNCH();
}

int fbam_adamw(void* param, const void* grad, float* m, float* v, float* master, long long n, int param_elem,
               float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
               void* stream) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 1023) / 1024);
  const uintptr_t pa = param_elem ? 7 : 15;
  const int vec_ok = !((reinterpret_cast<uintptr_t>(param) & pa) || (reinterpret_cast<uintptr_t>(grad) & pa) ||
                       (reinterpret_cast<uintptr_t>(m) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
                       (reinterpret_cast<uintptr_t>(master) & 15));
  if (param_elem)
    adamw_kernel<elem_t><<<blocks, 256, 0, STREAM(stream)>>>((elem_t*)param, (const elem_t*)grad, m, v, master, n, lr, b1, b2,
                                                           eps, wd, 1.0f / bc1, 1.0f / bc2, grad_scale, vec_ok);
  else
    adamw_kernel<float><<<blocks, 256, 0, STREAM(stream)>>>((float*)param, (const float*)grad, m, v, master, n, lr, b1,
                                                            b2, eps, wd, 1.0f / bc1, 1.0f / bc2, grad_scale, vec_ok);
  return CHECK_LAUNCH();
}

// velocity may be null (no momentum); master may be null (fp32 parameters).
int fbam_sgd(void* param, const void* grad, float* velocity, float* master, long long n, int param_elem, float lr,
             float momentum, int nesterov, float wd, void* stream) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (param_elem)
    sgd_kernel<elem_t><<<blocks, 256, 0, STREAM(stream)>>>((elem_t*)param, (const elem_t*)grad, velocity, master, n, lr,
                                                        momentum, nesterov, wd);
  else
    sgd_kernel<float><<<blocks, 256, 0, STREAM(stream)>>>((float*)param, (const float*)grad, velocity, master, n, lr,
                                                         momentum, nesterov, wd);
  return CHECK_LAUNCH();
}

// out: two zero-initialised 64-bit words in device memory; data must be 8-byte aligned.
int fbam_fingerprint(const void* data, long long n_bytes, unsigned long long* out, void* stream) {
  if (n_bytes < 0 || (reinterpret_cast<uintptr_t>(data) & 7) != 0) return 1;
  if (n_bytes == 0) return 0;
  const long long n_words = n_bytes / 8;
  const int tail = (int)(n_bytes % 8);
  long long blocks = (n_words + 256 * 8 - 1) / (256 * 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  fingerprint_kernel<<<(unsigned)blocks, 256, 0, STREAM(stream)>>>(
      (const unsigned long long*)data, n_words, (const unsigned char*)data + n_words * 8, tail, out);
  return CHECK_LAUNCH();
}

}  // extern "C"
