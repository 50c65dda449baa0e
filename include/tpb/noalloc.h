/* A C entry point for callers that must not allocate device memory.
 *
 * This function has no counterpart in the reference library; it exists for users of this one.
 *
 * Who it is for: code that runs where a cudaMalloc is off the table — a serving loop that cannot
 * afford the device-wide synchronisation an allocation or free implies, a plugin that was handed a
 * fixed memory budget and does not own an allocator, a process whose framework has already claimed
 * the whole GPU for its caching pool, or a signal/teardown path where allocating is simply unsafe.
 * Such callers still want to move a handful of buffers with one fused launch and get a
 * release-ordered completion flag, which normally needs a little device scratch memory (the table
 * of copies and the counter the thread blocks arrive on).
 *
 * What it does: copies `count` byte ranges (any alignment, local or peer-mapped destinations) with a
 * single kernel launch on `stream`, then — if `flag` is not NULL — stores `flag_value` to `*flag`
 * with release semantics at system scope once every byte is visible. The result is the same as
 * calling the library's ordinary push kernel for the same ranges.
 *
 * Where the scratch lives: in a fixed array inside the library image (device memory that every GPU
 * which loads this library holds until the process exits: 256 bytes of counters plus
 * TPB_NOALLOC_MAX_ITEMS table entries, about 8 KiB). Nothing is allocated or freed by this call,
 * and no allocating library routine is used.
 *
 * Rules that follow from sharing one array:
 *   - `count` may not exceed TPB_NOALLOC_MAX_ITEMS; larger requests are refused with
 *     TPB_NOALLOC_TOO_MANY (split them over several calls on the same stream).
 *   - Calls are safe back to back on ONE stream. Two calls whose kernels could overlap on a GPU
 *     (different streams, or different threads launching at once) race on the array: serialise them.
 *   - The array keeps whatever the previous call left in it; each call clears the counter it needs
 *     and rewrites the table before its kernel runs, in stream order.
 *   - The first call on each device looks up the array's device address (with that device current).
 *     Make that first call before starting any stream capture.
 *
 * Returns TPB_NOALLOC_OK (0) or a negative code; tpb_noalloc_strerror() explains a code.
 */
#ifndef TPB_NOALLOC_H_
#define TPB_NOALLOC_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TPB_NOALLOC_MAX_ITEMS 256

enum {
  TPB_NOALLOC_OK = 0,
  TPB_NOALLOC_TOO_MANY = -1,    /* count > TPB_NOALLOC_MAX_ITEMS */
  TPB_NOALLOC_BAD_ARGUMENT = -2,
  TPB_NOALLOC_CUDA_ERROR = -3   /* a CUDA runtime call failed; see tpb_noalloc_strerror */
};

typedef struct tpb_noalloc_item {
  const void* src;
  void* dst;
  uint64_t bytes;
} tpb_noalloc_item;

/* `stream` is a cudaStream_t. The current device must be the one that owns the stream. */
int tpb_noalloc_push(const tpb_noalloc_item* items, size_t count, uint32_t* flag, uint32_t flag_value,
                     void* stream);

/* Human-readable text for a return code (for TPB_NOALLOC_CUDA_ERROR: the last CUDA error text seen
 * by the calling thread). The pointer stays valid until the thread's next failing call. */
const char* tpb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* TPB_NOALLOC_H_ */
