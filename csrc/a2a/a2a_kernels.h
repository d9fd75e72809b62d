// Launchers of the dispatch / combine kernels (implemented in a2a_kernels.cu).
// Counterpart of the reference's p2p-all-to-all/a2a-kernels/src/a2a/a2a_kernels.h:17-141,
// with structs instead of ~30 positional pointers per call.
#pragma once

#include <cuda_runtime.h>

#include "a2a_types.h"

namespace pplx {

// Threads that cooperate on one token/record (32, 128 or 512) when `work_items` items of
// `vectors_per_item` 16-byte vectors each are spread over the grid.
int a2a_pick_team(const A2AConfig& cfg, int64_t work_items, int64_t vectors_per_item);

// `nranks` > 1 plays that many virtual ranks in one launch on the current device.
// A team size of 0 skips that phase; otherwise it is 32, 128 or 512.
cudaError_t a2a_launch_dispatch(const A2AConfig& cfg, const A2ARankStates& states, int nranks,
                                const PerRank<DispatchSendArgs>& send,
                                const PerRank<DispatchRecvArgs>& recv, int send_team, int recv_team,
                                cudaStream_t stream);

// Loads every kernel a context with this configuration can launch, on the current device. With
// lazy module loading the first launch of a kernel may have to wait for the kernels that are
// running; a dispatch that is running may in turn be waiting for a peer whose next kernel is
// that first launch. Loading at set-up time takes the first launches out of the steady state.
cudaError_t a2a_preload_kernels(const A2AConfig& cfg);

// All ranks of the context meet on the device (bounded wait, reported through the status word).
cudaError_t a2a_launch_barrier(const A2AConfig& cfg, const A2ARankStates& states, int nranks,
                               cudaStream_t stream);

cudaError_t a2a_launch_combine(const A2AConfig& cfg, const A2ARankStates& states, int nranks,
                               const PerRank<CombineSendArgs>& send,
                               const PerRank<CombineRecvArgs>& recv, int send_team, int recv_team,
                               int y_dtype, int out_dtype, cudaStream_t stream);

}  // namespace pplx
