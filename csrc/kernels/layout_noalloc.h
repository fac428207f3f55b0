/* Allocation-free entry point of the routing-layout kernel.
 *
 * This function has no counterpart in the reference library; it exists for callers that must not allocate
 * device memory when they ask for a routing layout: a serving process that sized all of its memory up front
 * and runs with no headroom, a plugin loaded into a host program that owns the allocator and forbids calls
 * into it from foreign code, or a latency-critical loop in which an allocation (and the implicit device
 * synchronisation a fresh `cudaMalloc` can cause) is not acceptable. The regular Python/C++ entry point
 * (`get_dispatch_layout`) obtains its scratch block from the PyTorch allocator on every call; this one keeps the
 * scratch block in a fixed array inside the loaded library instead.
 *
 * What the caller passes: the inputs and the three output arrays, all in device memory of the current device.
 * What the library holds: one `LayoutScratch` block (about 17 KB) and one status word per GPU that loads the
 * library, for the life of the process.
 *
 * Limits (requests outside them are rejected with DEEP_EP_NOALLOC_BAD_ARGUMENT, nothing is launched and the
 * outputs are left untouched):
 *   1 <= num_tokens <= DEEP_EP_NOALLOC_MAX_TOKENS (1,048,576); an empty batch is rejected too, unlike the regular
 *        entry point: a caller with no tokens clears its two count arrays itself
 *   num_topk    <= 32, num_experts <= 2048, num_ranks <= 64, num_experts % num_ranks == 0
 *
 * Behaviour to know about:
 *   - The first call on each device looks up the device address of the scratch array. Make that first call
 *     outside of any stream capture, with the device that will run the kernel current.
 *   - All calls on one device share the scratch array. Two calls whose kernels may overlap on the GPU (different
 *     streams without an ordering between them) race on it and give wrong results; order them.
 *   - The scratch block is cleared on the given stream before every launch, so a previous call's contents (or a
 *     previous call that failed half-way) never leak into the next one.
 *   - The return code covers the host side only (arguments, launch). The kernel synchronises its thread blocks with
 *     a wait that gives up after 10 seconds (it never spins for ever); if that happens the outputs are incomplete.
 *     The kernel records it in a status word that deep_ep_noalloc_wait_status() reads back, so a caller that wants
 *     certainty calls that function before it uses the outputs.
 *   - No cudaMalloc/cudaFree, no PyTorch allocation and no other allocating library routine is called.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define DEEP_EP_NOALLOC_OK 0
#define DEEP_EP_NOALLOC_BAD_ARGUMENT 1      /* null pointer, non-positive size, or a size beyond the limits above */
#define DEEP_EP_NOALLOC_CUDA_ERROR 2        /* a CUDA runtime call failed; see deep_ep_noalloc_last_error() */
#define DEEP_EP_NOALLOC_MAX_TOKENS (1 << 20)

/* Computes dst_slot_idx [num_tokens, num_topk], num_tokens_per_rank [num_ranks] and
 * num_tokens_per_expert [num_experts] (all int32, device memory) from topk_idx [num_tokens, num_topk] (int64,
 * device memory, -1 = no selection). `stream` is a cudaStream_t (0 = default stream). Returns one of the
 * DEEP_EP_NOALLOC_* codes; the work is enqueued on `stream`, not waited for. */
int deep_ep_dispatch_layout_noalloc(const long long* topk_idx, int num_tokens, int num_topk, int num_experts,
                                    int num_ranks, int* dst_slot_idx, int* num_tokens_per_rank,
                                    int* num_tokens_per_expert, void* stream);

/* Waits for `stream` and writes to `*device_status` how the most recent layout kernel on the current device ended:
 * 0 = it ran to completion, anything else = a wait inside the kernel ran out and the outputs are incomplete. The word
 * belongs to the device, not to a call: read it before the next deep_ep_dispatch_layout_noalloc() on that device.
 * Returns DEEP_EP_NOALLOC_OK when the word could be read. Allocates nothing; synchronises `stream`. */
int deep_ep_noalloc_wait_status(void* stream, int* device_status);

/* Text of the last failure reported by the functions above in this thread ("" if none). */
const char* deep_ep_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
