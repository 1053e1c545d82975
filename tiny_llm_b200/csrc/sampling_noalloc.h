// tllm_sample_noalloc: next-token sampling for callers that must not allocate device memory.
//
// This entry point has no counterpart in zscey/tiny-llm (whose sampling runs on the CPU and whose
// device buffers all come from its own allocator); it exists for users of this library.
//
// Who needs it.  tllm_sample() wants n * V floats of scratch from its caller.  Some callers cannot
// provide them: code that runs inside a region where the CUDA allocator may not be entered (a
// latency-critical serving loop that has pinned its memory budget up front, a plugin called from a
// host application that owns the device's memory pool, a callback running while another thread
// holds the allocator's lock), or a thin C client that links this library without any tensor
// runtime and simply has no scratch to hand over.  For them the scratch lives inside the library,
// in a file-scope __device__ array of TLLM_SAMPLE_NOALLOC_MAX_FLOATS floats (4 MiB).  Every GPU that
// loads the library holds that array until the process exits.
//
// Contract.
//   * Same arguments and the same result as tllm_sample(), minus the scratch pointer.
//   * n * V must not exceed TLLM_SAMPLE_NOALLOC_MAX_FLOATS; a larger request is refused with
//     TLLM_ERR_ARG (-1) and a message in tllm_last_error().  Nothing is launched then.
//   * The call performs no cudaMalloc, cudaFree or other allocating call.
//   * The first call on each device resolves the array's device address (cudaGetSymbolAddress, with
//     that device current).  Make that first call outside of any stream capture.
//   * All calls share the one array.  It keeps whatever the last call left in it; the kernel
//     writes every element of a row before it reads it, so nothing has to start at zero.  Two calls
//     that overlap on the GPU (different streams, no ordering between them) race on the array: order
//     them yourself.
#pragma once

#define TLLM_SAMPLE_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// logits: float32 [n, V] on the current device.  temperature, top_k, top_p, seeds, counters: device
// arrays of n entries (a row with temperature <= 0 is taken greedily).  out: int32 [n] on the device.
// stream: a cudaStream_t.  Returns 0, or a negative code with a message in tllm_last_error().
int tllm_sample_noalloc(const float* logits, int n, int v, const float* temperature, const int* top_k,
                        const float* top_p, const unsigned long long* seeds, const unsigned long long* counters,
                        int* out, void* stream);

#ifdef __cplusplus
}
#endif
