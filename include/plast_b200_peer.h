/*
 * plast_b200_peer.h — the exchange step of reductions that cross GPUs, over NVLink peer memory.
 *
 * The reference has no multi-GPU layer, so nothing here replaces a reference interface. The hot
 * path shards across the GPUs of one box along the outermost kept dim; full reductions, column
 * sums of a row-sharded matrix, the cross-entropy mean and bias gradients then need ONE exchange
 * of a tiny partial (4 bytes to 32 KiB). A library all-reduce costs 25-35 us for such a message on
 * eight GPUs, several times the local kernel; here every rank stores its partial straight into
 * every peer's exchange buffer (peer-to-peer stores over NVLink, 8-byte packets that carry the
 * value and the call's sequence number, so no fence and no separate flag), polls its own buffer
 * for the packets of the others and adds the values up in rank order — one small kernel,
 * identical bits on every rank. One process per GPU; buffers are shared through CUDA IPC handles that the
 * caller passes between the processes (64 opaque bytes per rank, by any transport).
 */
#ifndef PLAST_B200_PEER_H
#define PLAST_B200_PEER_H

#include "plast_b200.h"

#define PLAST_B200_IPC_HANDLE_BYTES 64
#define PLAST_B200_PEER_MAX_WORLD 8
#define PLAST_B200_PEER_MAX_FLOATS 8192 /* largest message of one exchange (32 KiB) */

#define PLAST_B200_PEER_SUM 0
#define PLAST_B200_PEER_MAX 1
#define PLAST_B200_PEER_MIN 2

/* plast_b200_peer_group_status value for "the local part of a fused call failed on this rank":
 * the rank still made its call of the exchange sequence, with an invalid contribution. */
#define PLAST_B200_PEER_STATUS_LOCAL_FAILURE 0x100

#ifdef __cplusplus
extern "C" {
#endif

typedef struct PlastPeerGroup PlastPeerGroup;

/* Step 1, on every rank: allocates this rank's exchange buffer on the current device (zeroed) and
 * writes its IPC handle. Returns NULL on failure (see plast_b200_last_error). */
PlastPeerGroup *plast_b200_peer_group_begin(int rank, int world, unsigned char handle[PLAST_B200_IPC_HANDLE_BYTES]);
/* Step 2, after the caller gathered every rank's handle (world x 64 bytes, in rank order) and ALL
 * ranks have completed step 1: maps the peers' buffers. Returns 0 on success. The caller then runs
 * a barrier of its own before the first exchange (a rank must not store into a buffer whose owner
 * has not finished step 1). */
int plast_b200_peer_group_connect(PlastPeerGroup *group, const unsigned char *all_handles);
/* In-place all-reduce of n <= PLAST_B200_PEER_MAX_FLOATS floats at `data` (device memory of this
 * rank) on the library stream; every rank must make the same sequence of calls. The partials are
 * combined in rank order, so every rank ends with the same bits. Waits inside the kernel are
 * bounded (about a second): if a peer never arrives the kernel gives up, the data is left
 * unreduced and plast_b200_peer_group_status reports it; nothing hangs. */
void plast_b200_peer_all_reduce(PlastPeerGroup *group, float *data, u64 n, int op);
/* The full reduction (op = PLAST_B200_PEER_SUM / MAX / MIN over every element of `input`, this
 * rank's shard) and the exchange of its result as ONE kernel: output->data[0] receives the value
 * over all ranks' shards. Counts as one call of the exchange sequence (every rank calls it at the
 * same point). For a mean, divide the sum by the global element count. */
void plast_b200_peer_full_reduce(PlastPeerGroup *group, int op, const Tensor *input, Tensor *output);
/* Mean cross-entropy over row-sharded logits (this rank holds `logits` [rows_here, C] and their
 * INT32 `labels`; global_rows = rows over all ranks): the loss sums of the ranks are exchanged
 * inside the cross-entropy kernel and divided by global_rows; output->data[0] receives the same
 * mean on every rank. One call of the exchange sequence. */
void plast_b200_peer_cross_entropy_mean(PlastPeerGroup *group, const Tensor *logits, const Tensor *labels,
                                        Tensor *output, u64 global_rows);
/* Bracket for reductions that cross the sharded dim. Every final reduction that entry points called
 * by THIS host thread launch between _begin and _end is combined across the ranks, in launch order:
 * a forward sum / max / min over the sharded axis (the column sum of a row-sharded matrix), the
 * broadcast-gradient reduce of a backward call (the bias / scale gradient of a batch-sharded
 * activation: inputs[i]->grad += the sum over ALL ranks' shards). Where the reduction kernel ends
 * with one thread or one row of strip owners holding the final values (full reductions, column
 * reductions onto contiguous outputs) the exchange happens inside that kernel; any other shape is
 * followed by the stand-alone exchange kernel on a parked copy, so the result is the same either
 * way and each reduction is exactly one call of the exchange sequence. Every rank must issue the
 * same calls in the same order. Limits: at most PLAST_B200_PEER_MAX_FLOATS contiguous outputs per
 * reduction; sum, max and min only (a mean would divide by the local count: take the sum and divide
 * by the global count), otherwise the call fails with PLAST_B200_ERR_UNSUPPORTED and launches
 * nothing. _end returns the number of exchanges made since _begin (0 means the bracketed calls
 * contained no reduction). */
void plast_b200_peer_reduce_begin(PlastPeerGroup *group);
int plast_b200_peer_reduce_end(PlastPeerGroup *group);
/* 0 = every exchange so far completed; 1 <= k <= world: a wait for rank k - 1 ran out;
 * PLAST_B200_PEER_STATUS_LOCAL_FAILURE: a fused call's local kernel could not run here (see
 * plast_b200_last_error at that call) and the exchanged value is invalid. Sticky until
 * plast_b200_peer_group_clear_status. Synchronises the library stream. */
int plast_b200_peer_group_status(PlastPeerGroup *group);
void plast_b200_peer_group_clear_status(PlastPeerGroup *group);
/* Unmaps the peers and frees this rank's buffer. Every rank calls it after its last exchange has
 * completed on every rank (barrier first). */
void plast_b200_peer_group_release(PlastPeerGroup *group);

/* Test hooks. A group whose `world` ranks all live in THIS process, rank 0 being the caller and
 * the others plain local buffers that nobody signals: with world == 1 the exchange completes by
 * itself; with world > 1 the wait for rank 1 runs out after `max_spins` polls (the bounded-wait
 * path, exercised without a second GPU and without hanging anything). */
PlastPeerGroup *plast_b200_peer_group_local(int world, unsigned max_spins);

#ifdef __cplusplus
}
#endif

#endif /* PLAST_B200_PEER_H */
