// Allocation-free entry point for the persistent LSTM forward kernel.
//
// This entry point has no counterpart in the reference trainer; it exists for callers of this library that
// are not allowed to allocate device memory at the point where they run the recurrence.  Typical cases: a
// host that owns the whole device heap and hands this library only the input and output buffers (an
// embedding runtime with a fixed memory plan); code running between the begin and end of a region in which
// the allocator is frozen; or a process whose memory budget was fully committed at start-up, where a
// cudaMalloc could fail or stall the device.  Such callers cannot provide the two pieces of scratch the
// kernel needs (the double-buffered h vector the CTAs exchange each step, and the grid-barrier counter), so
// the library keeps them in a fixed device array that is part of the loaded module.
//
// Contract
//   * Same arguments and results as fbam_lstm_fwd, minus the scratch pointers: `gates` (T, B, 4H) fp32 holds the
//     gate pre-activations (input projection + biases) on entry and the activated gates on exit; `y` (T, B, H)
//     bf16 and `c_all` (T, B, H) fp32 are outputs; `whh` is (4H, H) bf16; `h0`, `c0` are (H) fp32; `status` is a
//     caller-provided device word that receives a code if a bounded wait inside the kernel expires.
//   * Limits: H <= FBAM_LSTM_NOALLOC_MAX_HIDDEN, H a multiple of 16, 1 <= B <= 8.  Anything larger is refused
//     with FBAM_LSTM_NOALLOC_ERR_TOO_LARGE (see fbam_lstm_fwd_noalloc_strerror) and nothing is launched.
//   * The scratch array (FBAM_LSTM_NOALLOC_SCRATCH_BYTES, about 33 KB) lives in every device that loads the
//     library, from load until the process exits.
//   * The first call on a device looks up the array's device address (one-time set-up for that device, done
//     with that device current).  Make that first call outside any stream capture.  The looked-up address is
//     published through an atomic slot per device, so first calls from several host threads are safe.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any call.
//   * All calls on a device share the one array.  The barrier counter is cleared at the start of every call; the
//     h buffer is fully rewritten before it is read.  Two calls that overlap on the GPU (different streams, or
//     different host threads) would race on the array: serialise them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define FBAM_LSTM_NOALLOC_MAX_HIDDEN 1024
#define FBAM_LSTM_NOALLOC_SCRATCH_BYTES (2 * 8 * FBAM_LSTM_NOALLOC_MAX_HIDDEN * 2 + 256)
#define FBAM_LSTM_NOALLOC_ERR_TOO_LARGE 401
#define FBAM_LSTM_NOALLOC_ERR_SETUP 402

int fbam_lstm_fwd_noalloc(float* gates, const void* whh, const float* h0, const float* c0, void* y, float* c_all,
                          int* status, int T, int B, int H, void* stream);
int fbam_lstm_fwd_noalloc_max_hidden(void);
const char* fbam_lstm_fwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
