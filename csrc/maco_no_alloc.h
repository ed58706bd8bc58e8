// Entry point for callers that may not allocate device memory.
//
// This has no counterpart in the reference project.
//
// Some callers cannot call cudaMalloc (or anything that may call it for them, a framework's caching
// allocator included) at the moment they need decode attention: code that runs with a fixed,
// pre-sized memory plan, a serving loop that must not touch the allocator between requests because
// an allocation can synchronise the device or fail under fragmentation, or a plug-in that is handed
// tensors but no allocator. maco_attention_decode() needs a scratch buffer for its split-KV
// partial results, which such a caller cannot provide.
//
// maco_attention_decode_static() is the same computation with that scratch placed in a fixed
// array inside the library's device image:
//
//   * The array is MACO_STATIC_SCRATCH_BYTES (4 MiB) large. Every GPU that loads the library
//     holds it from load until the process exits, whether or not this function is ever called.
//   * A call needs  B * Hkv * splits * (G*128 + 2*G) * 4  bytes of it  (G = Hq / Hkv). A call
//     that needs more is refused with a non-zero return code and a message in maco_last_error();
//     nothing is launched. Use fewer splits, or the allocating entry point.
//   * The function itself calls no cudaMalloc / cudaFree and no library routine that allocates.
//     The first call on each device looks up the array's device address (once per device, with
//     that device current). Make that first call outside of any stream capture.
//   * All calls on a device share the one array, and it keeps whatever the previous call left in
//     it. Nothing in it has to start at zero: every partial a call reads was written by that same
//     call earlier on the same stream. Two calls whose kernels overlap on the GPU (different
//     streams, no ordering between them) race on the array and corrupt each other's results;
//     order them on one stream or with events.
//
// Inputs and outputs are the caller's, exactly as for maco_attention_decode():
//   q [B, Hq, 128], k / v [B, Hkv, S, 128] (16-bit, rows contiguous), out [B, Hq, 128].
// Returns 0 on success.
#pragma once

#define MACO_STATIC_SCRATCH_BYTES (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int maco_attention_decode_static(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hkv,
                                 int S, int head_dim, int splits, int dtype, long long kv_batch_stride,
                                 long long kv_head_stride, float scale, void* stream);

#ifdef __cplusplus
}
#endif
