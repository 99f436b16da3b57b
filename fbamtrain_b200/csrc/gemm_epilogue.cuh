// Fused epilogue shared by the tcgen05 GEMM kernels: one call handles 32 consecutive output columns of one row.
#pragma once
#include "gemm_tcgen05.h"
#include "gelu_math.cuh"
#include "elem16.cuh"

// The row-store variant of the reduce-scatter epilogue (GemmParams::rs_row_stores) is compiled in only on request
// (-DFBAM_RS_ROW_STORES=1, `FBAMTRAIN_RS_ROW_STORES=1 python -m fbamtrain_b200.build --force`): it raises the
// register count of every kernel that includes this epilogue, and until it has been measured the default build
// keeps the kernels exactly as they were profiled.  Without it the flag is ignored (default store pattern).
#ifndef FBAM_RS_ROW_STORES
#define FBAM_RS_ROW_STORES 0
#endif

namespace gemm_epi {

// GELU and gelu' come from gelu_math.cuh (packed fp32 pairs): the epilogue must not cost more issue slots than the
// tile's main loop, which erff() — and, for short K, even a scalar polynomial form — would.
__device__ __forceinline__ float gelu_f(float x) { return gelu_math::gelu1(x); }
__device__ __forceinline__ float gelu_grad_f(float x) { return gelu_math::gelu_grad1(x); }

__device__ __forceinline__ uint4 shfl_xor_u4(const uint4& x, int lane_mask) {
  uint4 y;
  y.x = __shfl_xor_sync(0xffffffffu, x.x, lane_mask);
  y.y = __shfl_xor_sync(0xffffffffu, x.y, lane_mask);
  y.z = __shfl_xor_sync(0xffffffffu, x.z, lane_mask);
  y.w = __shfl_xor_sync(0xffffffffu, x.w, lane_mask);
  return y;
}

// The epilogue reads at most one bf16 side input per element that is worth fetching a chunk ahead: the
// pre-activation whose GELU derivative scales the result, or else the residual.  aux_row_ptr gives that input's row
// (null when there is none, or when it cannot be read with 16-byte loads); aux_prefetch issues the four loads of
// columns [n0, n0 + 32) so that their latency passes while the previous chunk is converted and stored.
__device__ __forceinline__ const elem_t* aux_row_ptr(const GemmParams& p, long long roff) {
  if (roff < 0 || !p.vec_ok) return nullptr;
  if (p.gelu_grad_in != nullptr) return p.gelu_grad_in + roff;
  if (p.residual != nullptr && (p.ldr % 8 == 0)) return p.residual + roff / p.ldd * p.ldr;
  return nullptr;
}

__device__ __forceinline__ void aux_prefetch(const elem_t* aux_row, int n0, int n_total, uint4 (&aux)[4]) {
  if (aux_row != nullptr && n0 + 32 <= n_total) {
#pragma unroll
    for (int q = 0; q < 4; ++q) aux[q] = *reinterpret_cast<const uint4*>(aux_row + n0 + 8 * q);
  }
}

// Staging for TMA stores: a lane writes the four 16-byte pieces of its row's 64-byte chunk into a 32-row x 64-byte
// buffer in the layout of CU_TENSOR_MAP_SWIZZLE_64B (piece index XOR bits 1-2 of the row), which also keeps the
// writes of a warp free of bank conflicts.  The buffer must be 512-byte aligned.
__device__ __forceinline__ void stage_row64(uint8_t* buffer, const float (&v)[32]) {
  const int lane = threadIdx.x & 31;
  uint4* row = reinterpret_cast<uint4*>(buffer + lane * 64);
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __align__(16) elem2_t h[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) h[q] = ff2e2(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
    row[j ^ sw] = *reinterpret_cast<uint4*>(h);
  }
}

// r: 32 fp32 accumulator values of output row `roff / ldd`, columns [n0, n0 + 32).  With PRE, `pre` holds what
// aux_prefetch loaded for this chunk (valid whenever the chunk takes the vector path).  With STAGE (16-bit output
// without accumulation, a full 32-column chunk; every lane of the warp calls, lanes whose row is outside the output
// with roff < 0) nothing is stored to global memory: the result goes to `stage_out` and the pre-activation, if
// requested, to `stage_pre`, for the caller's TMA stores (which clip rows outside the output).
template <bool CE = false, bool PRE = false, bool STAGE = false>
__device__ __forceinline__ void store_chunk(const GemmParams& p, long long roff, int n0, const uint32_t (&r)[32],
                                            const uint4 (&pre)[4], uint8_t* stage_pre = nullptr,
                                            uint8_t* stage_out = nullptr) {
          const bool valid = roff >= 0;
          if (!STAGE && !valid) return;
          float v[32];
  #pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          if constexpr (CE) {
            if (p.ce_mode == 2 && valid) {   // logits -> scale * (softmax - onehot), straight from the accumulators
              const long long m = roff / p.ldd;
              const float lse = p.ce_lse[m];
              const int tgt = (int)p.ce_targets[m];
  #pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = n0 + j;
                const float sm = __expf(v[j] - lse) - (col == tgt ? 1.0f : 0.0f);
                v[j] = col < p.ce_vocab ? p.ce_scale * sm : 0.0f;
              }
            }
          }
          const bool full_vec = (n0 + 32 <= p.N) && p.vec_ok;
          if (p.bias != nullptr) {
            // every lane of the warp needs the same 32 bias values: 16-byte loads (served by L1 after the first tile)
            // instead of 32 scalar ones, whenever the chunk is whole and the vector is 16-byte aligned
            if (n0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
              if (p.bias_fp32) {
                const float4* b4 = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.bias) + n0);
  #pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const float4 t = __ldg(b4 + q);
                  v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
                }
              } else {
                const uint4* b4 = reinterpret_cast<const uint4*>(reinterpret_cast<const elem_t*>(p.bias) + n0);
  #pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 raw = __ldg(b4 + q);
                  const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
  #pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = e22ff(h[e]);
                    v[8 * q + 2 * e] += f.x;
                    v[8 * q + 2 * e + 1] += f.y;
                  }
                }
              }
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N)
                  v[j] += p.bias_fp32 ? reinterpret_cast<const float*>(p.bias)[n0 + j]
                                      : e2f(reinterpret_cast<const elem_t*>(p.bias)[n0 + j]);
            }
          }
          if (p.preact_out != nullptr) {
            elem_t* po = p.preact_out + roff + n0;
            if constexpr (STAGE) {
              stage_row64(stage_pre, v);
            } else if (full_vec) {
  #pragma unroll
              for (int j = 0; j < 32; j += 8) {
                __align__(16) elem2_t h[4];
  #pragma unroll
                for (int q = 0; q < 4; ++q) h[q] = ff2e2(v[j + 2 * q], v[j + 2 * q + 1]);
                *reinterpret_cast<uint4*>(po + j) = *reinterpret_cast<uint4*>(h);
              }
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) po[j] = f2e(v[j]);
            }
          }
          if (p.act == GEMM_ACT_GELU) {
  #pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float2 g = gelu_math::gelu2(make_float2(v[j], v[j + 1]));
              v[j] = g.x;
              v[j + 1] = g.y;
            }
          } else if (p.act == GEMM_ACT_RELU) {
  #pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
          }
          if (p.gelu_grad_in != nullptr) {
            const elem_t* gi = p.gelu_grad_in + roff + n0;
            if (full_vec) {
  #pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 raw;
                if constexpr (PRE) raw = pre[j / 8];
                else raw = valid ? *reinterpret_cast<const uint4*>(gi + j) : make_uint4(0, 0, 0, 0);
                const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
  #pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float2 g = gelu_math::gelu_grad2(e22ff(h[q]));
                  v[j + 2 * q] *= g.x;
                  v[j + 2 * q + 1] *= g.y;
                }
              }
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) v[j] *= gelu_grad_f(e2f(gi[j]));
            }
          }
          if (p.residual != nullptr) {
            const elem_t* ri = p.residual + roff / p.ldd * p.ldr + n0;
            if (full_vec && (p.ldr % 8 == 0)) {
  #pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 raw;
                if (PRE && p.gelu_grad_in == nullptr) raw = pre[j / 8];
                else raw = valid ? *reinterpret_cast<const uint4*>(ri + j) : make_uint4(0, 0, 0, 0);
                const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
  #pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float2 f = e22ff(h[q]);
                  v[j + 2 * q] += f.x;
                  v[j + 2 * q + 1] += f.y;
                }
              }
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (valid && n0 + j < p.N) v[j] += e2f(ri[j]);
            }
          }
          if constexpr (STAGE) {
            stage_row64(stage_out, v);
            return;
          }
          if (p.rs_rows_per_rank > 0 && p.rs_slot_plus1 > 0) {
            // GEMM -> reduce-scatter, slot form: this rank's partial tile goes, as bf16, into its slot of the
            // owner's buffer (plain 16-byte stores over NVLink)
            const int m = (int)(roff / p.ldd);
            const int owner = m / p.rs_rows_per_rank;
            elem_t* out = reinterpret_cast<elem_t*>(p.rs_out[owner]) +
                                 ((long long)(p.rs_slot_plus1 - 1) * p.rs_rows_per_rank + (m - owner * p.rs_rows_per_rank)) *
                                     p.ldd + n0;
#if FBAM_RS_ROW_STORES
            if (full_vec && p.rs_row_stores != 0 && (p.M & 31) == 0 && (p.rs_rows_per_rank & 31) == 0) {
              // Every lane of the warp is here (rows of a warp are 32 consecutive ones and M is a multiple of 32),
              // and the four rows of a lane quad belong to the same owner.  4 x 4 transpose of the 16-byte pieces
              // inside each quad: afterwards lane j of the quad holds piece j of the quad's rows 0..3.
              uint4 piece[4];
  #pragma unroll
              for (int q = 0; q < 4; ++q) {
                __align__(16) elem2_t h[4];
  #pragma unroll
                for (int e = 0; e < 4; ++e) h[e] = ff2e2(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
                piece[q] = *reinterpret_cast<uint4*>(h);
              }
              const int j = (int)(threadIdx.x & 3);
  #pragma unroll
              for (int k = 0; k < 4; k += 2) {        // exchange with the neighbouring lane
                const uint4 send = (j & 1) ? piece[k] : piece[k + 1];
                const uint4 got = shfl_xor_u4(send, 1);
                if (j & 1) piece[k] = got; else piece[k + 1] = got;
              }
  #pragma unroll
              for (int b = 0; b < 2; ++b) {           // exchange with the lane two further
                const uint4 send = (j & 2) ? piece[b] : piece[2 + b];
                const uint4 got = shfl_xor_u4(send, 2);
                if (j & 2) piece[b] = got; else piece[2 + b] = got;
              }
  #pragma unroll
              for (int q = 0; q < 4; ++q)             // row (own row - j + q), columns [n0 + 8j, n0 + 8j + 8)
                *reinterpret_cast<uint4*>(out + (long long)(q - j) * p.ldd + 8 * j) = piece[q];
            } else
#endif
            if (full_vec) {
  #pragma unroll
              for (int j = 0; j < 32; j += 8) {
                __align__(16) elem2_t h[4];
  #pragma unroll
                for (int q = 0; q < 4; ++q) h[q] = ff2e2(v[j + 2 * q], v[j + 2 * q + 1]);
                *reinterpret_cast<uint4*>(out + j) = *reinterpret_cast<uint4*>(h);
              }
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) out[j] = f2e(v[j]);
            }
            return;
          }
          if (p.rs_rows_per_rank > 0) {
            // GEMM -> reduce-scatter: add this rank's partial sums into the owner's fp32 buffer over NVLink
            const int m = (int)(roff / p.ldd);
            const int owner = m / p.rs_rows_per_rank;
            float* out = reinterpret_cast<float*>(p.rs_out[owner]) + (long long)(m - owner * p.rs_rows_per_rank) * p.ldd + n0;
            if (full_vec) {
  #pragma unroll
              for (int j = 0; j < 32; j += 4)
                asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + j), "f"(v[j]),
                             "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3])
                             : "memory");
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N)
                  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(out + j), "f"(v[j]) : "memory");
            }
            return;
          }
          if (p.out_fp32) {
            float* out = reinterpret_cast<float*>(p.D) + roff + n0;
            if (p.accumulate == GEMM_ACC_ATOMIC) {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) atomicAdd(out + j, v[j]);
            } else if (full_vec) {
  #pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (p.accumulate) {
                  float4 c = *reinterpret_cast<const float4*>(out + j);
                  o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
                }
                *reinterpret_cast<float4*>(out + j) = o;
              }
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) out[j] = p.accumulate ? out[j] + v[j] : v[j];
            }
          } else {
            elem_t* out = reinterpret_cast<elem_t*>(p.D) + roff + n0;
            if (full_vec) {
  #pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (p.accumulate) {
                  uint4 raw = *reinterpret_cast<const uint4*>(out + j);
                  const elem2_t* h = reinterpret_cast<const elem2_t*>(&raw);
  #pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    float2 f = e22ff(h[q]);
                    v[j + 2 * q] += f.x;
                    v[j + 2 * q + 1] += f.y;
                  }
                }
                __align__(16) elem2_t h[4];
  #pragma unroll
                for (int q = 0; q < 4; ++q) h[q] = ff2e2(v[j + 2 * q], v[j + 2 * q + 1]);
                *reinterpret_cast<uint4*>(out + j) = *reinterpret_cast<uint4*>(h);
              }
            } else {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N)
                  out[j] = f2e(p.accumulate ? e2f(out[j]) + v[j] : v[j]);
            }
          }

}

template <bool CE = false>
__device__ __forceinline__ void store_chunk(const GemmParams& p, long long roff, int n0, const uint32_t (&r)[32]) {
  const uint4 none[4] = {};
  store_chunk<CE, false>(p, roff, n0, r, none);
}

}  // namespace gemm_epi
