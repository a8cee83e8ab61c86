/*
 * exchange_b200.h - C ABI of the one exchange step of a sharded engine step: the all-gather of the
 * sampled token ids.
 *
 * Sequences and their KV block pools are partitioned by rank, so the attention operator and the
 * sampler need no collective; after Sampler::sample (src/cpp/src/sampling/sampler.cpp:1708-1810)
 * every rank's scheduler must see every sequence's new token before it plans the next step
 * (src/cpp/src/continuous_batching/pipeline_impl.cpp:378-533 is single-process: there the ids are
 * simply in host memory).  The reference has no multi-device counterpart of this call.
 *
 * Layout: one device buffer of [world][cap] int64, rank-contiguous.  Rank r's sampler writes its n_r
 * ids (n_r <= cap) straight into row r (exchange_b200_local_row), then ONE ncclAllGather, in place,
 * on the stream the sampler ran on, fills the other rows.  Which sequence a slot belongs to is host
 * knowledge (the partition), not data that travels.  Unused slots hold -1.
 *
 * NCCL is bound at run time (dlopen of libnccl.so.2: inside a process that has PyTorch loaded this is
 * PyTorch's copy), so the library itself loads on machines without NCCL.
 */
#ifndef EXCHANGE_B200_H
#define EXCHANGE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EXCHANGE_B200_ID_BYTES 128

typedef enum exchange_status {
    EXCHANGE_OK = 0,
    EXCHANGE_ERR_INVALID_ARG = 1,
    EXCHANGE_ERR_NO_NCCL = 2, /* libnccl.so.2 or one of its symbols could not be bound */
    EXCHANGE_ERR_NCCL = 3,    /* an NCCL call failed; see exchange_b200_last_error()   */
    EXCHANGE_ERR_CUDA = 4
} exchange_status;

typedef struct exchange_handle exchange_handle;

const char* exchange_b200_last_error(void);

/* Rank 0 makes the communicator id (ncclGetUniqueId); the caller hands the bytes to the other ranks
 * by whatever control channel it has (the scheduler's own, MPI, a torch.distributed broadcast). */
int exchange_b200_unique_id(uint8_t id[EXCHANGE_B200_ID_BYTES]);

/* Joins the communicator (collective over all ranks) and allocates the [world][cap] buffer. */
int exchange_b200_create(const uint8_t id[EXCHANGE_B200_ID_BYTES], int32_t rank, int32_t world, int32_t device, int32_t cap,
                         exchange_handle** out);
int exchange_b200_destroy(exchange_handle* h);

/* Device pointers: this rank's row of the buffer (the sampler's out_token for this step) and the whole buffer. */
int64_t* exchange_b200_local_row(exchange_handle* h);
int64_t* exchange_b200_all_rows(exchange_handle* h);

/* Marks the slots of the local row from n_local on as unused (-1) and all-gathers the rows in place.
 * Asynchronous on `stream` (a cudaStream_t; NULL = the default stream).  One NCCL call, no host copy. */
int exchange_b200_all_gather_ids(exchange_handle* h, int32_t n_local, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EXCHANGE_B200_H */
