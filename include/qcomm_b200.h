/* qcomm_b200 -- one-shot all-reduce (sum) of small 16-bit vectors over NVLink peer memory.
 *
 * Tensor-parallel decode of the packed models splits o_proj / down_proj along K: every rank produces
 * a partial [M, hidden] result (16 - 64 KB) that must be summed over the ranks, 2 x layers times per
 * token.  At that size a collective is pure latency, so this one is a single kernel per rank:
 * every rank stores its vector into a slot of EVERY rank's receive buffer over NVLink / NVSwitch as
 * self-validating 8-byte words -- 4 bytes of data and the 32-bit tag of the call; an aligned 8-byte
 * store arrives whole, so whoever sees the tag has the data, and there is no fence, no separate
 * flag and no second trip over the link -- then polls its own buffer, a bounded time, until the
 * words of all ranks carry the call's tag, and adds them in rank order (fp32 accumulation), so that
 * all ranks compute bit-identical sums.  Two buffer halves alternate from call to call; a rank
 * cannot run two calls ahead of another, so nothing is overwritten while it is still being read.
 * That is the protocol for two ranks.  From three ranks up every thread would have to poll every
 * peer, and the older protocol measures faster: plain 16-byte stores into the slots, a system-wide
 * fence, one flag per (rank, CTA) raised with a release store, one polling thread per peer, then the
 * sum (8 GPUs, 70B-shape decode: 131 against 118 tok/s).  qcomm_allreduce picks by the group's size;
 * qcomm_allreduce_rmsnorm always uses data + flags.  The two protocols have their own parts of the buffers.
 *
 * Peer loads and stores only: no in-switch reduction or broadcast, no library kernel is handed a peer pointer.
 * The reference project has no multi-GPU path, so nothing here has a counterpart in it; the
 * contract is the all-reduce of a Megatron-style K-split Linear.
 *
 * Same conventions as qgemv_b200.h: plain pointers and sizes, negative QGEMV_ERR_* codes,
 * qgemv_error_string() for the last error.  Set-up calls (qcomm_alloc, qcomm_ipc_*) allocate or map
 * device memory and may synchronise; qcomm_allreduce only launches a kernel.
 */
#ifndef QCOMM_B200_H
#define QCOMM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QCOMM_MAX_RANKS 8
#define QCOMM_MAX_BLOCKS 64              /* CTAs per call; 4096 elements each */
#define QCOMM_IPC_HANDLE_BYTES 64

/* One rank's view of the group.  slots[r] / flags[r] are rank r's receive areas as addressable from
 * THIS process (r == rank: local memory; otherwise a peer mapping).  All areas are zero-initialised
 * once at set-up and never cleared afterwards. */
typedef struct qcomm_group {
    int32_t rank, world;                 /* 1 <= world <= QCOMM_MAX_RANKS */
    int32_t max_elems;                   /* capacity of one slot in 16-bit elements, multiple of 8 */
    int32_t wait_limit;                  /* probes of a flag before giving up; 0 = default (about a second) */
    void* slots[QCOMM_MAX_RANKS];        /* each qcomm_slot_bytes(world, max_elems): [2 halves][world][max_elems] x 16 bit of plain
                                            data, then [2 halves][world][max_elems / 2] tagged 8-byte words */
    void* flags[QCOMM_MAX_RANKS];        /* each qcomm_flag_bytes(world): [2 halves][world][QCOMM_MAX_BLOCKS] uint32 */
    void* state;                         /* local, 256 bytes: call counter, finished-CTA counter, status word */
} qcomm_group;

size_t qcomm_slot_bytes(int world, int max_elems);
size_t qcomm_flag_bytes(int world);
size_t qcomm_state_bytes(void);

/* data[i] <- sum over ranks of their data[i], i < elems, in place, on `stream`.  `data` is local
 * device memory, 16-byte aligned; elems is a multiple of 8 and at most max_elems; dtype is QGEMV_F16
 * or QGEMV_BF16.  Every rank of the group must issue the same sequence of calls.  Capturable in a
 * CUDA graph (the call counter lives in device memory).  The kernel waits for the preceding kernel
 * of the stream before it reads `data` and lets the following one start early (programmatic
 * dependent launch).  If a peer's words do not arrive within the wait limit the kernel finishes
 * anyway, with whatever the slot holds, and raises the status word. */
int qcomm_allreduce(const qcomm_group* g, void* data, int64_t elems, int dtype, void* stream);

/* The all-reduce fused with the step that follows it in a decoder layer -- residual update and RMS
 * normalisation -- as ONE kernel (one CTA per row):
 *     d[m, :]  = r(sum over ranks of their partial[m, :])      (rounded as a separate all-reduce would store it)
 *     h[m, :] <- r(h[m, :] + d[m, :])                          (in place)
 *     y[m, :]  = r(weight[:] * r(h[m, :] * rsqrt(mean(h[m, :]^2) + eps)))
 * partial: this rank's [rows, hidden] partial result of a K-split projection (leading dimension ldp);
 * h, y, weight as in qdec_rmsnorm (qdecode_b200.h).  rows <= QCOMM_MAX_BLOCKS, hidden a multiple of 8
 * and at most 16384, rows * hidden <= max_elems, all rows 16-byte aligned.  Counts as one call of
 * the group's call sequence, like qcomm_allreduce; same waiting and status behaviour. */
int qcomm_allreduce_rmsnorm(const qcomm_group* g, const void* partial, int64_t ldp, void* h, int64_t ldh,
                            const void* weight, void* y, int64_t ldy, int rows, int hidden, float eps,
                            int dtype, void* stream);

/* Enqueue a copy of the status word into *host_out (0 = every call so far completed; 1 = a wait for
 * a peer ran out) and reset it; synchronise `stream` before reading. */
int qcomm_status(const qcomm_group* g, void* stream, int32_t* host_out);

/* Set-up helpers: zero-filled device memory that can be shared with the other ranks of the node, its
 * inter-process handle (QCOMM_IPC_HANDLE_BYTES bytes, to be sent to the peers by any host channel),
 * and the mapping of a peer's handle into this process (enables peer access). */
int qcomm_alloc(size_t bytes, void** dev_ptr);
int qcomm_free(void* dev_ptr);
int qcomm_ipc_export(void* dev_ptr, void* handle_out);
int qcomm_ipc_open(const void* handle, void** dev_ptr);
int qcomm_ipc_close(void* dev_ptr);

#ifdef __cplusplus
}
#endif
#endif /* QCOMM_B200_H */
