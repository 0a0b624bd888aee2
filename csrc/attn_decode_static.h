// Split-K decode attention that needs no scratch buffer from its caller and allocates nothing.
//
// This entry point has no counterpart in the reference engine; it exists for callers of the C ABI that cannot
// allocate device memory at the moment they need attention: code running between the begin and end of a stream
// capture, a host thread that does not own an allocator (a plug-in that is handed raw pointers by another
// framework), or a process that has already handed all free device memory to its KV cache.  zse_attn_decode asks
// such a caller for `zse_attn_decode_scratch_floats(...)` floats of scratch when num_splits > 1; this variant keeps
// the scratch in a fixed array that is part of the library image on every device.
//
// Limit.  The array holds ZSE_ATTN_STATIC_SCRATCH_FLOATS floats (16 MiB).  A call needs
// num_seqs * nh * num_splits * (hd + 2) floats when num_splits > 1 and none when num_splits == 1; a call that needs
// more returns ZSE_ERR_LIMIT and launches nothing.  zse_attn_decode_static_max_floats() returns the limit so that a
// caller can choose a smaller num_splits up front.
//
// Set-up.  The first call on each device looks the array's address up (cudaGetSymbolAddress) and remembers it; that
// lookup is host work, may synchronise with the device, and is not a stream operation; the same goes for the kernel's
// shared-memory attribute, which is raised once per device.  zse_attn_decode_static_setup() does both for the current
// device: call it on each device before the first call that is part of a stream capture, and from ONE host thread -
// the per-device records are filled without a lock, so the first use of a device is not thread-safe (two threads
// racing there write the same values, but nothing guarantees it).  A failed lookup returns ZSE_ERR_DRIVER and is
// retried by the next call.  A call with num_splits == 1 needs no scratch and does no lookup.
//
// Sharing.  Every call on one device uses the same array.  Nothing in it has to start at zero: each call writes
// every word it later reads.  Two calls that may run at the same time on one device (different streams without an
// ordering between them) race on the array and produce wrong results; order them on one stream or with events.
#pragma once
#include <stdint.h>

#define ZSE_ATTN_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int64_t zse_attn_decode_static_max_floats(void);
// looks the scratch array up and raises the kernels' shared-memory attribute on the current device; 0 or an error code
int zse_attn_decode_static_setup(void);
// same arguments and results as zse_attn_decode, minus the scratch pointer
int zse_attn_decode_static(const void* q, int ldq, const void* kv_layer, const void* block_tables_i32, int max_blocks,
                           const void* seq_lens_i32, void* out_f16, int ldo, int num_seqs, int nh, int nkv, int hd,
                           int block_size, int num_splits, float scale, void* stream);

#ifdef __cplusplus
}
#endif
