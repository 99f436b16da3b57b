// Store-pattern micro-benchmark: how fast can 148 SMs write an [M x 256] 16-bit matrix (512-byte rows), depending on
// which lanes of a warp write which bytes?
//   mode 0: one ROW per lane, four 16-byte stores per 64-byte chunk (what a tensor-memory epilogue does when every
//           lane stores its own accumulator row from registers): each store instruction touches 32 rows.
//   mode 1: one row per warp instruction (32 lanes x 16 bytes = the whole 512-byte row).
//   mode 2: eight rows x 64 bytes per instruction (four neighbouring lanes cover one row's chunk).
// Build and run:  nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o store_pattern benchmarks/store_pattern.cu && ./store_pattern
// Measured on a B200: mode 0 tops out at 2.6 TB/s, modes 1 and 2 reach 6.2 TB/s (memset 6.9 TB/s) - which is why the
// GEMM / convolution epilogues stage their tiles in shared memory and write them with TMA tiled stores.
#include <cstdio>
#include <cuda_runtime.h>
#include <cstdint>
template <int MODE>
__global__ void k(uint4* out, long long rows, int warps_per_cta) {
  // tiles of 128 rows x 256 cols (512 B per row); warp w: lane group w%4 -> rows 32*(w%4)+lane, column part w/4
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int parts = warps_per_cta / 4;            // column parts per row (2 -> 128 cols each, 4 -> 64 cols each)
  const int part = warp / 4, lg = warp % 4;
  const long long tiles = rows / 128;
  for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
    const long long row = t * 128 + lg * 32 + lane;
    const int pieces = 32 / parts;               // 16-byte pieces per thread per row
    if (MODE == 0) {                              // row per lane, 4 x 16 B per chunk
      uint4* p = out + row * 32 + part * pieces;
      for (int c = 0; c < pieces; c += 4) {
        uint4 v = make_uint4(c, lane, warp, (unsigned)t);
#pragma unroll
        for (int q = 0; q < 4; ++q) p[c + q] = v;
      }
    } else if (MODE == 1) {                       // full rows: each warp instruction writes one 512-byte row
      // warp handles rows lg*32 .. +32 of its column part... for the comparison let every warp write whole rows
      for (int r = part; r < 32; r += parts) {
        const long long rr = t * 128 + lg * 32 + r;
        out[rr * 32 + lane] = make_uint4(r, lane, warp, (unsigned)t);
      }
    } else {                                      // 8 rows x 64 B per instruction
      for (int c = 0; c < pieces; c += 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long rr = t * 128 + lg * 32 + j * 8 + (lane >> 2);
          out[rr * 32 + part * pieces + c + (lane & 3)] = make_uint4(c, lane, warp, (unsigned)t);
        }
      }
    }
  }
}
int main() {
  const long long rows = 1966080;
  uint4* out; cudaMalloc(&out, rows * 512);
  char* flush; cudaMalloc(&flush, 256 << 20);
  cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
  for (int mode = 0; mode < 3; ++mode)
    for (int warps : {8, 16})
      for (int ctas : {148, 296, 592}) {
        float best = 1e9;
        for (int it = 0; it < 6; ++it) {
          cudaMemset(flush, 0, 256 << 20);
          cudaEventRecord(a);
          if (mode == 0) k<0><<<ctas, warps * 32>>>(out, rows, warps);
          if (mode == 1) k<1><<<ctas, warps * 32>>>(out, rows, warps);
          if (mode == 2) k<2><<<ctas, warps * 32>>>(out, rows, warps);
          cudaEventRecord(b); cudaEventSynchronize(b);
          float ms; cudaEventElapsedTime(&ms, a, b);
          if (it >= 2 && ms < best) best = ms;
        }
        printf("mode %d warps %2d ctas %3d: %.3f ms  %.0f GB/s\n", mode, warps, ctas, best, rows * 512 / best / 1e6);
      }
  cudaEventRecord(a); cudaMemsetAsync(out, 0, rows * 512); cudaEventRecord(b); cudaEventSynchronize(b);
  float ms; cudaEventElapsedTime(&ms, a, b); printf("memset %.3f ms %.0f GB/s\n", ms, rows * 512 / ms / 1e6);
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}
