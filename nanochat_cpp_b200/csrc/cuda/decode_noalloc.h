// A C entry point for paged decode attention that allocates no memory at all.
//
// This function has no counterpart in the reference implementation. It exists for callers that must not
// allocate while they run a decode step: a serving process that has handed all of the device's memory to its
// own pool (so a driver allocation may fail, and an allocation or free through the driver can stall every
// stream of the device while it happens), a host application in another language that reaches this library
// through its C symbols and has no tensor allocator to lend, and latency-critical loops that have to know
// that a call is a kernel launch and nothing else. The tensor-level entry point (`paged_decode_attention` of
// the Python extension) obtains the output tensor and, when the keys are split over several CTAs, two scratch
// tensors from the framework's allocator on every call; this one takes the output from the caller and keeps the
// scratch in a fixed array that is part of the loaded library.
//
// Scratch and its limit
//   The array holds NC_DECODE_NOALLOC_MAX_FLOATS floats (8 MiB). It is a file-scope device array, so every
//   GPU on which this library is loaded holds those 8 MiB until the process exits, whether or not the
//   function is ever called. A call needs B * H * splits * (D + 2) floats of it when splits > 1 and none when
//   splits == 1; a call that would need more is refused with NC_DECODE_NOALLOC_TOO_LARGE and launches nothing.
//
// Set-up
//   The first call on a device looks up the device address of the array (once per device, with that device
//   current) and remembers it. Make that first call outside of any stream capture; later calls only launch.
//   The caller selects the device (cudaSetDevice) before calling; all pointers belong to that device.
//
// Sharing
//   All calls on a device share the one array and it keeps whatever the last call left in it. Nothing in it
//   has to start at zero: every slot that the combine step reads is written by the same call before. Two
//   calls that overlap on the GPU (different streams, or different host threads on different streams) race
//   on the array and produce garbage; calls on one stream are ordered and safe.
//
// Results are identical to the tensor-level entry point for the same `splits`.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define NC_DECODE_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)

enum {
  NC_DECODE_NOALLOC_OK = 0,
  NC_DECODE_NOALLOC_BAD_ARGUMENT = 1,  // null or misaligned pointer, unsupported head size or group size (H / KV not
                                       // in {1, 2, 4, 8}), non-positive counts, max_pages * page_size > INT_MAX
  NC_DECODE_NOALLOC_TOO_LARGE = 2,     // the scratch array cannot hold B * H * splits * (D + 2) floats
  NC_DECODE_NOALLOC_CUDA_ERROR = 3,    // set-up or the launch failed; see the message
};

// q, out:            bf16 [B, H, D], contiguous
// k_pool, v_pool:    bf16 [pages, page_size, KV, D]
// page_table:        int32 [B, max_pages]; seq_lens: int32 [B], counting the token that is being decoded. The entry
//                    point cannot read device memory without a synchronisation, so it does not validate the
//                    lengths: the kernel clamps a length above max_pages * page_size to that bound (the table is
//                    never indexed out of range) and skips a sequence whose length is <= 0. Page numbers inside
//                    the table are the caller's responsibility.
// q, k_pool, v_pool, out must be 16-byte aligned (the kernels use 16-byte loads and stores).
// window_left:       keys further back than this are not attended; negative = unlimited
// splits:            CTAs per (sequence, kv head) along the keys; <= 0 picks the value the tensor-level entry
//                    point would pick for these sizes
// stream:            a cudaStream_t (null = the default stream)
// message:           optional buffer that receives a description of a failure
// Returns one of the NC_DECODE_NOALLOC_* codes.
__attribute__((visibility("default"))) int nc_paged_decode_attention_noalloc(
    const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_lens, void* out,
    int B, int H, int KV, int D, int max_pages, int page_size, int window_left, float scale, int splits,
    void* stream, char* message, int message_len);

// The number of key splits the tensor-level entry point uses for these sizes.
__attribute__((visibility("default"))) int nc_paged_decode_attention_splits(int B, int KV, int max_pages,
                                                                             int page_size, int window_left);

#ifdef __cplusplus
}
#endif
