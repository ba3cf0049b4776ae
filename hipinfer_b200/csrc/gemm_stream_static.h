// hb_gemm_stream_static: the decode-step matrix product for callers that cannot allocate.
//
// This entry point has no counterpart in the reference project; it exists for users of this
// library only.
//
// Who needs it: code that runs where device memory must not be requested. Examples are a
// plug-in inside a host application that owns all of the GPU's memory and hands out none, a
// caller on a real-time or signal-handling path where cudaMalloc (which may synchronise the
// device and take a driver lock) is forbidden, and a process that was started with a fixed
// memory budget that is already spent. hb_gemm_stream needs a workspace for split-K partial
// sums and a few counters, which its caller normally allocates; this variant keeps both in
// two arrays that are part of the library's own device image, so it calls no cudaMalloc,
// cudaFree or any routine that allocates (none of PyTorch's either).
//
//   C (+)= A W^T,  A [M, K] bf16 (row stride lda), W [N, K] bf16 (row stride ldw), M <= 64,
//   K a multiple of 8; C and `epi` as for hb_gemm_stream (0 fp32 store, 1 bf16 store,
//   2 add into fp32, 3 SwiGLU to bf16 [M, N/2]); `status` a device-visible int that is set to 1
//   if a bounded wait inside the kernel ran out.
//
// Limits. The scratch array holds HB_STATIC_WS_FLOATS floats (4 MiB) and the counter array
// HB_STATIC_COUNTERS ints; every GPU that loads the library carries them until the process
// exits. A product whose split needs more (the message states how much) is refused with -1 and
// a text in hb_last_error(); nothing is launched then.
//
// Rules for the caller.
//  * The first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress,
//    with that device current). Make that first call outside any CUDA stream capture.
//  * All calls share the two arrays and each call finds what the previous one left. The call
//    clears the counters it is going to use (a cudaMemsetAsync on `stream`); the partial sums
//    need no clearing because every slot that is read was written by the same call.
//  * Calls that overlap on the GPU (issued to different streams, or from several host threads
//    at once) race on the arrays. Issue them to one stream, one after the other.
#pragma once
#include <cuda_runtime.h>

#define HB_STATIC_WS_FLOATS (1 << 20)
#define HB_STATIC_COUNTERS 1024
#define HB_STATIC_MAX_DEVICES 64

extern "C" __attribute__((visibility("default"))) int hb_gemm_stream_static(const void* A, long lda, const void* W,
                                                                            long ldw, void* C, long ldc, int M, int N,
                                                                            int K, int epi, int* status,
                                                                            cudaStream_t stream);
