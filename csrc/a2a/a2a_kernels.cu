// Expert-parallel dispatch / combine kernels for one NVSwitch domain (sm_100a).
//
// Four phases, launched separately or fused pairwise (send+recv in one launch):
//
//   dispatch_send  per-expert counts -> peers first; then tokens -> peer receive regions
//                  (16-byte peer stores over NVLink), each record published by writing its
//                  tag last with release semantics
//   dispatch_recv  wait for the counts only, build the expert-major layout, then take the
//                  records one by one as their tags appear and replicate each into the
//                  rows of its local experts
//   combine_send   expert outputs -> origin ranks' combine regions; each row bumps the
//                  arrival counter of its token at the origin (release)
//   combine_recv   per token: wait for its rows, top-k weighted reduction into the
//                  caller's tensor
//
// They cover what the reference does with four cooperative kernels plus a host proxy
// thread (p2p-all-to-all/a2a-kernels/src/a2a/a2a_dispatch_send.cu:112-536,
// a2a_dispatch_recv.cu:16-236, a2a_combine_send.cu:20-235, a2a_combine_recv.cu:20-167,
// p2p-all-to-all/src/a2a_worker.rs:340-455), but the protocol is different:
//   * no CPU takes part; counts, payload and signals all travel as peer stores,
//   * a token crosses NVLink once per destination *rank*, not once per route,
//   * receive regions are sized for the worst case, so there is no overflow/pull path,
//   * no grid-wide barrier: a block never waits for another block of its own GPU,
//   * arrival is per record and per token, never "everything from everybody": the receive
//     side works while the rest of the payload is still on the wire,
//   * every wait on a remote flag is bounded in time and reports through a status word.
//
// blockIdx.y selects a *virtual rank*: with gridDim.y == 1 the launch serves the one
// rank of this process; with gridDim.y == R one launch on one GPU plays R ranks whose
// "peer" pointers all live on that GPU (used to test the multi-rank protocol and to
// profile it on a single device).

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <type_traits>

#include "a2a_kernels.h"
#include "a2a_types.h"
#include "ptx.cuh"
#include "a2a_device.cuh"
#include "../ops/router.cuh"
#include "a2a_ll.cuh"

namespace pplx {
namespace {

// ---------------------------------------------------------------------------
// dispatch_send
// ---------------------------------------------------------------------------
// Dynamic shared memory of the dispatch kernel: [histogram / layout tables | staging of one
// quantised token per team (flagged-line format with fused quantisation only)].
__host__ __device__ inline size_t dispatch_stage_offset(const A2AConfig& cfg) {
  const size_t send = (cfg.num_experts + kMaxRanks) * sizeof(uint32_t);
  const size_t gl = static_cast<size_t>(cfg.num_groups) * cfg.experts_per_rank;
  const size_t recv = (2 * gl + 2 * cfg.experts_per_rank + 32) * sizeof(uint32_t);
  return ((send > recv ? send : recv) + 15) / 16 * 16;
}

// Top-k routing of token t by the calling warp (see ops/router.cuh); lane r < k gets the r-th
// expert and its weight.
__device__ __forceinline__ void route_token(const A2AConfig& cfg, const DispatchSendArgs& a, int t,
                                            uint32_t* expert, float* weight) {
  const size_t elem = a.logits_bf16 ? 2 : 4;
  const void* row = static_cast<const char*>(a.logits) + static_cast<size_t>(t) * a.logits_stride * elem;
  if (cfg.num_experts <= 128) {
    ops::route_token_warp<4>(row, a.logits_bf16 != 0, a.logits_bias, cfg.num_experts, cfg.topk, expert, weight);
  } else if (cfg.num_experts <= 256) {
    ops::route_token_warp<8>(row, a.logits_bf16 != 0, a.logits_bias, cfg.num_experts, cfg.topk, expert, weight);
  } else {
    ops::route_token_warp<16>(row, a.logits_bf16 != 0, a.logits_bias, cfg.num_experts, cfg.topk, expert, weight);
  }
}

// The counts message of one dispatch, sent by one whole block from a histogram in shared memory:
// per destination, how many records it will get from this rank and how many of them each of
// its experts takes. It also tells every rank that this rank has started the dispatch (and so
// has left its previous combine): a rank that has heard that from everybody may write the
// combine buffers again.
template <int WIRE>
__device__ void send_counts(const A2AConfig& cfg, const A2ARankState& st, const uint32_t* hist,
                            const uint32_t* nrec, uint32_t tag, uint32_t par) {
  const A2ALocal& ws = st.local;
  const int world = cfg.world;
  const int L = cfg.experts_per_rank;
  const int my_group = st.rank / cfg.dp_size;
  const int my_tp = st.rank % cfg.dp_size;
    if (has_remote(cfg) && threadIdx.x < world) {
      const bool served = static_cast<int>(threadIdx.x % cfg.dp_size) == my_tp;
      reinterpret_cast<volatile uint32_t*>(ws.proxy)[kProxyRecords + threadIdx.x] = served ? nrec[threadIdx.x] : 0u;
    }
    if constexpr (WIRE == kWireLL) {
      // Flagged lines, to every rank (zeros where this rank serves no records): no fence, and
      // the lines themselves tell the receiver that this rank has started the dispatch.
      const uint32_t per_dst = cfg.counts_stride / 4;  // physical vectors per (source, destination)
      for (uint32_t i = threadIdx.x; i < world * per_dst; i += blockDim.x) {
        const uint32_t d = i / per_dst, pv = i % per_dst;
        const bool served = static_cast<int>(d % cfg.dp_size) == my_tp;
        Vec16 v = {tag, tag, tag, tag};
        if (!ll_is_flag(pv)) {
          uint32_t word[4];
          #pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t wi = 4 * ll_logical(pv) + c;
            const uint32_t e = d * L + (wi - 1);
            word[c] = !served ? 0u : wi == 0 ? nrec[d] : (wi <= static_cast<uint32_t>(L) && e < static_cast<uint32_t>(cfg.num_experts)) ? hist[e] : 0u;
          }
          v = Vec16{word[0], word[1], word[2], word[3]};
        }
        uint8_t* dst = st.sync[d] + cfg.off_counts +
                       4ull * (par * cfg.counts_bank_words + st.rank * cfg.counts_stride) + 16ull * pv;
        st_stream_v4(dst, v);
      }
    } else {
    const int per_dst = L + 1;
    for (int i = threadIdx.x; i < world * per_dst; i += blockDim.x) {
      const int d = i / per_dst;
      const int j = i % per_dst;
      if (d % cfg.dp_size != my_tp) continue;
      uint32_t v;
      if (j == 0) {
        v = nrec[d];
      } else {
        const int e = d * L + (j - 1);
        v = e < cfg.num_experts ? hist[e] : 0u;
      }
      uint32_t* dst = reinterpret_cast<uint32_t*>(st.sync[d] + cfg.off_counts) +
                      par * cfg.counts_bank_words + my_group * cfg.counts_stride + j;
      st_stream_u32(dst, v);
    }
    __syncthreads();
    if (threadIdx.x < world) {
      st_release_sys(flag_ptr(st.sync[threadIdx.x], kFlagDispatchStarted, st.rank), tag);
    }
    }  // plain wire
}

// Routing fused into the dispatch: every team added its token's routes to a histogram in device
// memory. The block that finishes its tokens last sends the counts message from it and clears
// it for the dispatch after next. Called by all threads of every block.
template <int WIRE>
__device__ void route_finish(const A2AConfig& cfg, const A2ARankState& st, uint32_t* dyn_smem, uint32_t tag,
                             uint32_t par) {
  const A2ALocal& ws = st.local;
  __shared__ uint32_t s_last_router;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last_router = atom_acq_rel_gpu_add(&ws.route_done[par], 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (s_last_router == 0) return;
  uint32_t* hist = dyn_smem;                // [num_experts]
  uint32_t* nrec = hist + cfg.num_experts;  // [kMaxRanks]
  for (int i = threadIdx.x; i < cfg.num_experts; i += blockDim.x) {
    volatile uint32_t* g = &ws.route_hist[par * cfg.num_experts + i];
    hist[i] = *g;
    *g = 0;
  }
  if (threadIdx.x < kMaxRanks) {
    volatile uint32_t* g = &ws.route_nrec[par * kMaxRanks + threadIdx.x];
    nrec[threadIdx.x] = *g;
    *g = 0;
  }
  if (threadIdx.x == 0) ws.route_done[par] = 0;
  __syncthreads();
  send_counts<WIRE>(cfg, st, hist, nrec, tag, par);
}

template <int WIRE>
__device__ void dispatch_send_phase(const A2AConfig& cfg, const A2ARankState& st,
                                    const DispatchSendArgs& a, uint32_t* dyn_smem, const int TEAM) {
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  const int world = cfg.world;
  const int K = cfg.topk;
  const int L = cfg.experts_per_rank;
  const int my_group = st.rank / cfg.dp_size;
  const int my_tp = st.rank % cfg.dp_size;
  const uint32_t epoch = read_epoch(ws, 0);
  const uint32_t tag = epoch + 1;
  const uint32_t par = epoch & 1u;
  trace_mark(cfg, ws, kTraceSendStart);

  int T = a.num_tokens;
  if (a.bound_m != nullptr) T = min(T, *a.bound_m);
  T = max(0, min(T, cfg.max_num_tokens));

  // ---- counts message: leaves before any payload, from the block with the fewest tokens ----
  // Per destination: how many records it will get from this rank and how many of them each
  // of its experts takes. The "dispatch started" word goes to every rank (also to those this
  // rank serves no records): a rank that has seen it from everybody knows that all ranks
  // have left their previous combine, so the combine buffers may be written again.
  const bool fused_route = a.logits != nullptr;
  if (fused_route && blockIdx.x == gridDim.x - 1 && threadIdx.x < kMaxRanks) {
    ws.send_cursor[(par ^ 1u) * kMaxRanks + threadIdx.x] = 0;
  }
  if (!fused_route && blockIdx.x == gridDim.x - 1) {
    uint32_t* hist = dyn_smem;                // [num_experts]
    uint32_t* nrec = hist + cfg.num_experts;  // [kMaxRanks]
    for (int i = threadIdx.x; i < cfg.num_experts + kMaxRanks; i += blockDim.x) hist[i] = 0;
    // the slot cursors of the next dispatch; nobody touches that bank during this launch
    if (threadIdx.x < kMaxRanks) ws.send_cursor[(par ^ 1u) * kMaxRanks + threadIdx.x] = 0;
    __syncthreads();
    for (int t = threadIdx.x; t < T; t += blockDim.x) {
      uint32_t mask = 0;
      for (int k = 0; k < K; ++k) {
        const uint32_t e = a.indices[t * a.indices_stride + k];
        if (e < static_cast<uint32_t>(cfg.num_experts)) {
          atomicAdd(&hist[e], 1u);
          mask |= 1u << (e / L);
        } else {
          report(ws, kStatusBadExpertIndex, kPhaseDispatchSend, t, e);
        }
      }
      for (int d = 0; d < world; ++d) {
        if ((mask >> d) & 1u) atomicAdd(&nrec[d], 1u);
      }
    }
    __syncthreads();
    send_counts<WIRE>(cfg, st, hist, nrec, tag, par);
    if (cfg.trace && threadIdx.x == 0) ws.trace[kTraceSendSignalled] = globaltimer_ns();
  }

  // ---- token loop: one team per token ----
  if constexpr (WIRE == kWireLL) {
    uint8_t* side = reinterpret_cast<uint8_t*>(dyn_smem) + dispatch_stage_offset(cfg);
    dispatch_send_tokens_ll(cfg, st, a, T, tag, par, TEAM, side,
                            [&](int t, uint32_t* e, float* w) { route_token(cfg, a, t, e, w); });
  } else {
  __shared__ uint32_t s_idx[kMaxTeams][kMaxTopK];
  __shared__ float s_w[kMaxTeams][kMaxTopK];
  __shared__ uint32_t s_slot[kMaxTeams][kMaxRanks];
  __shared__ uint32_t* s_pend[kMaxTeams][kMaxPending];   // tags not yet published
  __shared__ uint32_t s_npend[kMaxTeams];
  if (threadIdx.x < kMaxTeams) s_npend[threadIdx.x] = 0;
  __syncthreads();
  const uint32_t nvec = cfg.d_payload_bytes / 16;
  const int hs = cfg.hidden_dim_scale;
  constexpr int U = kCopyUnroll;
  for (int t = team.id; t < T; t += team.count) {
    const uint8_t* src = a.x + static_cast<uint64_t>(t) * a.x_stride;
    // payload loads do not depend on the routing: issue them first
    Vec16 v[U];
    if (!a.quantize) {
      #pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t i = team.lane + u * TEAM;
        if (i < nvec) v[u] = ld_input_v4(src + 16ull * i);
      }
    }
    if (fused_route) {
      if (team.lane < 32) {
        uint32_t e;
        float w;
        route_token(cfg, a, t, &e, &w);
        if (team.lane < K) {
          s_idx[team.in_block][team.lane] = e;
          s_w[team.in_block][team.lane] = w;
          const_cast<uint32_t*>(a.indices)[t * a.indices_stride + team.lane] = e;
          const_cast<float*>(a.weights)[t * a.weights_stride + team.lane] = w;
          atom_relaxed_gpu_add(&ws.route_hist[par * cfg.num_experts + e], 1u);
        }
      }
    } else if (team.lane < K) {
      s_idx[team.in_block][team.lane] = a.indices[t * a.indices_stride + team.lane];
      s_w[team.in_block][team.lane] = a.weights[t * a.weights_stride + team.lane];
    }
    team.sync();
    // one slot per destination rank that owns at least one of the token's experts
    uint32_t my_slot = kNoSlot;
    if (team.lane < kMaxRanks) {
      const int d = team.lane;
      bool hit = false;
      if (d < world && d % cfg.dp_size == my_tp) {
        for (int k = 0; k < K; ++k) {
          const uint32_t e = s_idx[team.in_block][k];
          hit |= e < static_cast<uint32_t>(cfg.num_experts) && e / L == static_cast<uint32_t>(d);
        }
      }
      if (hit) {
        if (fused_route) atom_relaxed_gpu_add(&ws.route_nrec[par * kMaxRanks + d], 1u);
        my_slot = atom_relaxed_gpu_add(&ws.send_cursor[par * kMaxRanks + d], 1u);
        if (my_slot >= static_cast<uint32_t>(cfg.max_num_tokens)) {
          report(ws, kStatusRecordOverflow, kPhaseDispatchSend, d, my_slot);
          my_slot = kNoSlot;
        }
      }
      s_slot[team.in_block][d] = my_slot;
    }
    team.sync();
    if (t == 0) trace_mark(cfg, ws, kTraceSendSlots);
    uint8_t* rec[kMaxRanks];
    #pragma unroll
    for (int d = 0; d < kMaxRanks; ++d) {
      const uint32_t slot = s_slot[team.in_block][d];
      rec[d] = (d < world && slot != kNoSlot)
                   ? st.recv[d] + cfg.off_drecv + my_group * cfg.drecv_group_stride +
                         static_cast<uint64_t>(slot) * cfg.d_stride
                   : nullptr;
    }

    // header (without its tag) and, when the caller supplies them, the scales as 16-byte
    // stores: small stores cost a full NVLink packet each
    {
      const int hdr_vecs = cfg.d_header_bytes / 16;
      const int scale_vecs = (!a.quantize && hs > 0) ? cfg.d_scale_bytes / 16 : 0;
      const float* xs = reinterpret_cast<const float*>(a.x_scale);
      for (int vi = team.lane; vi < hdr_vecs + scale_vecs; vi += TEAM) {
        uint32_t word[4];
        uint32_t at;
        if (vi < hdr_vecs) {
          #pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int wi = 4 * vi + c;
            if (wi == 0) word[c] = 0;  // the tag is written last, by the release below
            else if (wi == 1) word[c] = static_cast<uint32_t>(t);
            else if (wi < 2 + K) word[c] = s_idx[team.in_block][wi - 2];
            else if (wi < 2 + 2 * K) word[c] = __float_as_uint(s_w[team.in_block][wi - 2 - K]);
            else word[c] = 0;
          }
          at = 16u * vi;
        } else {
          const int sv = vi - hdr_vecs;
          #pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int j = 4 * sv + c;
            word[c] = j < hs ? __float_as_uint(xs[t * a.x_scale_stride_token + j * a.x_scale_stride_elem]) : 0u;
          }
          at = cfg.d_header_bytes + cfg.d_payload_bytes + 16u * sv;
        }
        const Vec16 q = {word[0], word[1], word[2], word[3]};
        #pragma unroll
        for (int d = 0; d < kMaxRanks; ++d) {
          if (rec[d] != nullptr) st_stream_v4(rec[d] + at, q);
        }
      }
    }

    if (!a.quantize) {
      for (uint32_t i0 = team.lane; i0 < nvec; i0 += TEAM * U) {
        if (i0 != team.lane) {
          #pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * TEAM;
            if (i < nvec) v[u] = ld_input_v4(src + 16ull * i);
          }
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t i = i0 + u * TEAM;
          if (i < nvec) {
            #pragma unroll
            for (int d = 0; d < kMaxRanks; ++d) {
              if (rec[d] != nullptr) st_stream_v4(rec[d] + cfg.d_header_bytes + 16ull * i, v[u]);
            }
          }
        }
      }
    } else {
      // bf16 in, e4m3 + one fp32 scale per 128 elements out. Lane i converts elements
      // [16 i, 16 i + 16); lanes 8 j .. 8 j + 7 of a warp share scale j.
      const uint32_t warp_lane = threadIdx.x & 31u;
      const uint32_t lane_base = team.lane - warp_lane;
      for (uint32_t base = lane_base; base < nvec; base += TEAM) {
        const uint32_t i = base + warp_lane;
        const bool valid = i < nvec;
        Vec16 lo = {0, 0, 0, 0}, hi = {0, 0, 0, 0};
        if (valid) {
          lo = ld_input_v4(src + 32ull * i);
          hi = ld_input_v4(src + 32ull * i + 16);
        }
        float scale;
        const Vec16 q = quantize16(lo, hi, &scale, a.quantize == 2);
        if (valid) {
          #pragma unroll
          for (int d = 0; d < kMaxRanks; ++d) {
            if (rec[d] != nullptr) {
              st_stream_v4(rec[d] + cfg.d_header_bytes + 16ull * i, q);
              if ((i & 7u) == 0) {
                st_stream_u32(rec[d] + cfg.d_header_bytes + cfg.d_payload_bytes + 4 * (i >> 3),
                              __float_as_uint(scale));
              }
            }
          }
        }
      }
    }
    // The record is complete once every lane's stores are: the barrier makes them all
    // "observed" by the lane that publishes the tag, and the release orders them before it.
    // A release is a fence that waits for everything this SM has in flight, so tags are
    // published for a few tokens at a time: the first warp keeps the list.
    if (t == 0) trace_mark(cfg, ws, kTraceSendStored);
    team.sync();
    if (team.lane < 32) {
      uint32_t npend = s_npend[team.in_block];
      uint32_t* mine = nullptr;
      if (team.lane < kMaxRanks && my_slot != kNoSlot) {
        mine = reinterpret_cast<uint32_t*>(st.recv[team.lane] + cfg.off_drecv +
                                           my_group * cfg.drecv_group_stride +
                                           static_cast<uint64_t>(my_slot) * cfg.d_stride);
      }
      const uint32_t mask = __ballot_sync(0xffffffffu, mine != nullptr);
      if (mine != nullptr) s_pend[team.in_block][npend + __popc(mask & ((1u << team.lane) - 1u))] = mine;
      npend += __popc(mask);
      __syncwarp();
      const bool last = t + team.count >= T;
      if (last || npend + kMaxRanks > kMaxPending) {
        if (team.lane < npend) st_release_sys(s_pend[team.in_block][team.lane], tag);
        npend = 0;
        __syncwarp();
      }
      if (team.lane == 0) s_npend[team.in_block] = npend;
    }
    if (t == 0) trace_mark(cfg, ws, kTraceSendPublished);
  }
  }  // plain wire
  if (fused_route) route_finish<WIRE>(cfg, st, dyn_smem, tag, par);
  proxy_phase_done(cfg, ws, 0, tag);
  trace_mark(cfg, ws, kTraceSendLoopDone);
  trace_max(cfg, ws, kTraceSendLoopLast);
  if (threadIdx.x == 0 && blockIdx.x == 0) atomicAdd(&ws.stats[0], static_cast<unsigned long long>(T));
}

// ---------------------------------------------------------------------------
// dispatch_recv
// ---------------------------------------------------------------------------
template <int WIRE>
__device__ void dispatch_recv_phase(const A2AConfig& cfg, const A2ARankState& st,
                                    const DispatchRecvArgs& a, uint32_t* dyn_smem, const int TEAM) {
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  const int G = cfg.num_groups;
  const int K = cfg.topk;
  const int L = cfg.experts_per_rank;
  const int rank = st.rank;
  const uint32_t epoch = read_epoch(ws, 0);
  const uint32_t tag = epoch + 1;
  const uint32_t par = epoch & 1u;
  trace_mark(cfg, ws, kTraceRecvStart);

  __shared__ uint32_t s_abort;
  __shared__ uint32_t s_rec_prefix[kMaxRanks + 1];
  __shared__ uint32_t s_rows[kMaxTeams][kMaxTopK];
  __shared__ uint32_t s_unused[kMaxTeams][kMaxTopK];
  __shared__ uint32_t s_nrows[kMaxTeams];

  __shared__ uint32_t s_nrec[kMaxRanks];
  uint32_t* cnt = dyn_smem;           // [G][L]
  uint32_t* base = cnt + G * L;       // [G][L]  first row of (group, expert)
  uint32_t* total = base + G * L;     // [L]
  uint32_t* pad_off = total + L;      // [L]
  uint32_t* misc = pad_off + L;       // [0] padded row count
  const uint32_t pad = static_cast<uint32_t>(cfg.expert_padding);

  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  // The counts message of this dispatch from every rank (ranks of another tensor-parallel lane
  // send no counts here, only the fact that they have started). The status word is fetched
  // while the wait runs.
  if constexpr (WIRE == kWireLL) {
    const uint32_t per_src = cfg.counts_stride / 4;  // physical vectors per source rank
    const uint32_t total_pv = cfg.world * per_src;
    const uint8_t* lines = st.sync[rank] + cfg.off_counts + 4ull * par * cfg.counts_bank_words;
    const uint32_t warp_first = threadIdx.x & ~31u;
    for (uint32_t w0 = warp_first; w0 < total_pv; w0 += blockDim.x) {
      const uint32_t i = w0 + (threadIdx.x & 31u);
      Vec16 v[1];
      const bool ok = ll_load_lines<1>(
          v, tag, [&](int) { return lines + 16ull * i; }, [&](int) { return i < total_pv; },
          cfg.wait_limit_ns, ws.status);
      if (!ok) {
        if ((threadIdx.x & 31u) == 0) report(ws, kStatusWaitTimeout, kPhaseDispatchRecv, i / per_src, tag);
        s_abort = 1;
      } else if (i < total_pv) {
        const uint32_t src = i / per_src, pv = i % per_src;
        if (!ll_is_flag(pv) && static_cast<int>(src % cfg.dp_size) == rank % cfg.dp_size) {
          const uint32_t g = src / cfg.dp_size;
          const uint32_t word[4] = {v[0].x, v[0].y, v[0].z, v[0].w};
          #pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t wi = 4 * ll_logical(pv) + c;
            if (wi == 0) s_nrec[g] = min(word[c], static_cast<uint32_t>(cfg.max_num_tokens));
            else if (wi <= static_cast<uint32_t>(L)) cnt[g * L + (wi - 1)] = word[c];
          }
        }
      }
    }
    if (threadIdx.x == 0 && ws.status[0] != 0) s_abort = 1;
  } else {
    if (threadIdx.x < cfg.world) {
      uint64_t waited;
      const bool ok = wait_flag(flag_ptr(st.sync[rank], kFlagDispatchStarted, threadIdx.x), tag,
                                cfg.wait_limit_ns, &waited);
      if (!ok) {
        report(ws, kStatusWaitTimeout, kPhaseDispatchRecv, threadIdx.x, tag);
        s_abort = 1;
      }
      if (blockIdx.x == 0) atomicMax(&ws.stats[2], static_cast<unsigned long long>(waited));
    } else if (threadIdx.x == 32 && ws.status[0] != 0) {
      s_abort = 1;
    }
    __syncthreads();
    if (s_abort == 0) {
      const uint32_t* counts = reinterpret_cast<const uint32_t*>(st.sync[rank] + cfg.off_counts) +
                               par * cfg.counts_bank_words;
      for (int i = threadIdx.x; i < G * L; i += blockDim.x) {
        const int g = i / L, le = i % L;
        cnt[i] = ld_relaxed_sys(counts + g * cfg.counts_stride + 1 + le);
      }
      if (threadIdx.x < G) {
        s_nrec[threadIdx.x] = min(ld_relaxed_sys(counts + threadIdx.x * cfg.counts_stride),
                                  static_cast<uint32_t>(cfg.max_num_tokens));
      }
    }
  }
  __syncthreads();
  const bool abort = s_abort != 0;  // uniform across the block
  trace_mark(cfg, ws, kTraceRecvWaitDone);

  // ---- expert-major layout from the counts (every block computes it privately) ----
  if (!abort) {
    // records per source group, prefix-summed by the first warp
    if (threadIdx.x < 32) {
      const uint32_t n = threadIdx.x < G ? s_nrec[threadIdx.x] : 0u;
      uint32_t incl = n;
      #pragma unroll
      for (int o = 1; o < kMaxRanks; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (threadIdx.x >= o) incl += up;
      }
      // lane g holds the inclusive sum up to group g; entry g + 1 is "records before g + 1"
      if (threadIdx.x == 0) s_rec_prefix[0] = 0;
      if (threadIdx.x < kMaxRanks) s_rec_prefix[threadIdx.x + 1] = incl;
    }
    __syncthreads();
    // totals per expert, in parallel over the experts
    for (int j = threadIdx.x; j < L; j += blockDim.x) {
      uint32_t tot = 0;
      for (int g = 0; g < G; ++g) tot += cnt[g * L + j];
      total[j] = tot;
    }
    __syncthreads();
    // exclusive scan of the padded totals: the first warp, each lane a contiguous chunk
    if (threadIdx.x < 32) {
      const int per = (L + 31) / 32;
      const int lo = threadIdx.x * per;
      const int hi = min(lo + per, L);
      uint32_t sum = 0;
      for (int j = lo; j < hi; ++j) sum += (total[j] + pad - 1) / pad * pad;
      uint32_t incl = sum;
      #pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
        if (threadIdx.x >= o) incl += n;
      }
      uint32_t run = incl - sum;
      for (int j = lo; j < hi; ++j) {
        pad_off[j] = run;
        run += (total[j] + pad - 1) / pad * pad;
      }
      if (threadIdx.x == 31) misc[0] = incl;
    }
    __syncthreads();
    // first row of every (group, expert), in parallel over the pairs
    for (int i = threadIdx.x; i < G * L; i += blockDim.x) {
      const int g = i / L, j = i % L;
      uint32_t row = pad_off[j];
      for (int q = 0; q < g; ++q) row += cnt[q * L + j];
      base[i] = row;
    }
    __syncthreads();
    trace_mark(cfg, ws, kTraceRecvLayoutDone);

    const uint32_t padded_rows = misc[0];
    const uint32_t row_cap = a.out_rows ? min(a.out_rows, cfg.max_recv_rows) : cfg.max_recv_rows;
    if (blockIdx.x == 0) {
      for (int le = threadIdx.x; le < L; le += blockDim.x) {
        a.out_num_tokens[le] = static_cast<int32_t>(total[le]);
        ws.expert_meta[2 + le] = total[le];
        ws.expert_meta[2 + L + le] = pad_off[le];
        // rows that only exist as padding carry no source
        const uint32_t end = pad_off[le] + (total[le] + pad - 1) / pad * pad;
        for (uint32_t r = pad_off[le] + total[le]; r < end && r < cfg.max_recv_rows; ++r) {
          ws.row_src[r] = kNoSlot;
        }
      }
      if (has_remote(cfg) && threadIdx.x == 32) {
        // where the combine will stage the rows of each origin group that has members outside
        // the NVLink domain: one dense segment per group, in group order
        uint32_t first = 0;
        for (int g = 0; g < G; ++g) {
          uint32_t rows_g = 0;
          for (int le = 0; le < L; ++le) rows_g += cnt[g * L + le];
          reinterpret_cast<volatile uint32_t*>(ws.proxy)[kProxyRowBase + g] = first;
          ws.stage_cursor[g] = 0;
          first += rows_g;
        }
      }
      if (threadIdx.x == 0) {
        ws.expert_meta[0] = min(padded_rows, row_cap);
        ws.expert_meta[1] = s_rec_prefix[G];
        if (padded_rows > row_cap) {
          report(ws, kStatusRowOverflow, kPhaseDispatchRecv, padded_rows, row_cap);
        }
      }
    }

    // ---- record loop: one team per record, each consumed as soon as its tag is there ----
    if constexpr (WIRE == kWireLL) {
      RecvLayout lay{base, s_rec_prefix, row_cap};
      uint8_t* side = reinterpret_cast<uint8_t*>(dyn_smem) + dispatch_stage_offset(cfg);
      dispatch_recv_records_ll(cfg, st, a, lay, tag, par, TEAM, s_rows, s_unused, s_nrows, side);
    } else {
    const uint32_t nvec = cfg.d_payload_bytes / 16;
    const int hs = cfg.hidden_dim_scale;
    const uint32_t total_recs = s_rec_prefix[G];
    const uint8_t* drecv = st.recv[rank] + cfg.off_drecv;
    constexpr int U = kCopyUnroll;
    for (uint32_t r = team.id; r < total_recs; r += team.count) {
      int g = 0;
      #pragma unroll
      for (int j = 1; j < kMaxRanks; ++j) {
        if (j < G && r >= s_rec_prefix[j]) g = j;
      }
      const uint32_t s = r - s_rec_prefix[g];
      const uint8_t* rec =
          drecv + g * cfg.drecv_group_stride + static_cast<uint64_t>(s) * cfg.d_stride;
      const uint32_t* hdr = reinterpret_cast<const uint32_t*>(rec);
      if (team.lane < 32) {
        uint32_t ok = 1;
        if (team.lane == 0) {
          ok = wait_word(hdr, tag, true, cfg.wait_limit_ns, ws.status) ? 1u : 0u;
          if (!ok) report(ws, kStatusWaitTimeout, kPhaseDispatchRecv, g, r);
        }
        __syncwarp();  // lane 0's acquire now covers the whole warp's reads of the record
        ok = __shfl_sync(0xffffffffu, ok, 0);
        const int k = team.lane;
        uint32_t row = kNoSlot;
        const uint32_t t = ok ? ld_relaxed_sys(hdr + 1) : 0u;
        if (ok && t >= static_cast<uint32_t>(cfg.max_num_tokens)) {
          if (k == 0) report(ws, kStatusBadRecord, kPhaseDispatchRecv, g, t);
          ok = 0;
        }
        if (ok && k < K) {
          const uint32_t e = ld_relaxed_sys(hdr + 2 + k);
          if (e < static_cast<uint32_t>(cfg.num_experts) && e / L == static_cast<uint32_t>(rank)) {
            const int le = e - rank * L;
            row = base[g * L + le] +
                  atom_relaxed_gpu_add(&ws.place_cursor[par * (G * L) + g * L + le], 1u);
            if (row < row_cap) {
              ws.row_src[row] = g;
              ws.row_tk[row] = t * K + k;
            } else {
              row = kNoSlot;
            }
          }
          if (cfg.combine_mode == kCombinePreReduce) {
            ws.rec_rows[static_cast<uint64_t>(r) * K + k] = row;
            ws.rec_weights[static_cast<uint64_t>(r) * K + k] =
                __uint_as_float(ld_relaxed_sys(hdr + 2 + K + k));
            if (k == 0) {
              ws.rec_token[2 * r] = t;
              ws.rec_token[2 * r + 1] = g;
            }
          }
        }
        compact_warp(row != kNoSlot, row, 0u, s_rows[team.in_block], s_unused[team.in_block],
                     &s_nrows[team.in_block]);
        if (!ok && team.lane == 0) s_nrows[team.in_block] = kTeamAbort;
      }
      team.sync();
      if (r == 0) trace_mark(cfg, ws, kTraceRecvFirstTag);

      const uint32_t nrows = s_nrows[team.in_block];
      if (nrows == kTeamAbort) break;  // uniform across the team
      if (nrows != 0) {
        for (uint32_t i0 = team.lane; i0 < nvec; i0 += TEAM * U) {
          Vec16 v[U];
          #pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * TEAM;
            if (i < nvec) v[u] = ld_stream_v4(rec + cfg.d_header_bytes + 16ull * i);
          }
          for (uint32_t j = 0; j < nrows; ++j) {
            uint8_t* dst =
                a.out_x + static_cast<uint64_t>(s_rows[team.in_block][j]) * a.out_x_stride;
            #pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint32_t i = i0 + u * TEAM;
              if (i < nvec) st_stream_v4(dst + 16ull * i, v[u]);
            }
          }
        }
        if (hs > 0 && a.out_x_scale != nullptr) {
          float* os = reinterpret_cast<float*>(a.out_x_scale);
          for (int j = team.lane; j < hs; j += TEAM) {
            const uint32_t bits = ld_relaxed_sys(
                reinterpret_cast<const uint32_t*>(rec + cfg.d_header_bytes + cfg.d_payload_bytes) + j);
            for (uint32_t q = 0; q < nrows; ++q) {
              os[static_cast<int64_t>(s_rows[team.in_block][q]) * a.out_x_scale_stride_token +
                 j * a.out_x_scale_stride_elem] = __uint_as_float(bits);
            }
          }
        }
      }
      team.sync();
    }
    }  // plain wire
  }
  trace_mark(cfg, ws, kTraceRecvLoopDone);
  trace_max(cfg, ws, kTraceRecvLoopLast);
  finish_recv(cfg, ws, 0, epoch, kTraceRecvAllDone, false);
}

// ---------------------------------------------------------------------------
// combine_send
// ---------------------------------------------------------------------------

// Per-route mode: plain byte copy of each valid expert row to every member of the
// origin dp group. Pre-reduce mode: weighted partial sum per received record. Either way
// the team that wrote a row announces it at once on the arrival counter of the row's token
// at the origin, so the origin reduces token by token while other rows are still in flight.
template <int WIRE, typename Y>
__device__ void combine_send_phase(const A2AConfig& cfg, const A2ARankState& st,
                                   const CombineSendArgs& a, const int TEAM) {
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  const int K = cfg.topk;
  trace_mark(cfg, ws, kTraceCSendStart);

  __shared__ uint32_t s_healthy;
  __shared__ uint32_t s_rows[kMaxTeams][kMaxTopK];
  __shared__ uint32_t s_wbits[kMaxTeams][kMaxTopK];
  __shared__ uint32_t s_n[kMaxTeams];
  // Plain wire: a row is announced by adding one to its token's arrival counter at the origin,
  // with release semantics. A release is a fence that waits for everything the SM has in flight,
  // so the first warp of a team collects the counters of a few rows and releases them together.
  __shared__ uint32_t* s_pend[kMaxTeams][kMaxPending];
  __shared__ uint32_t s_npend[kMaxTeams];
  if (threadIdx.x < kMaxTeams) s_npend[threadIdx.x] = 0;
  // issued together with the status word, not after it: each is a cold miss
  const uint32_t tag_c = read_epoch(ws, 1) + 1;
  const uint32_t meta_rows = ws.expert_meta[0];
  const uint32_t meta_recs = ws.expert_meta[1];
  if (threadIdx.x == 0) s_healthy = ws.status[0] == 0 ? 1u : 0u;
  __syncthreads();
  const bool healthy = s_healthy != 0;
  // both are called by the whole team, after the barrier that follows a row's stores
  auto flush = [&]() {
    if (team.lane < 32) {
      const uint32_t npend = s_npend[team.in_block];
      __syncwarp();
      if (team.lane < npend) red_release_sys_add(s_pend[team.in_block][team.lane], 1u);
      if (team.lane == 0) s_npend[team.in_block] = 0;
      __syncwarp();
    }
  };
  auto announce = [&](uint32_t g, uint32_t t) {
    if (team.lane < 32) {
      const uint32_t npend = s_npend[team.in_block];
      __syncwarp();
      // members of the origin group outside the NVLink domain are told by the proxy instead
      const bool member = team.lane < cfg.dp_size && in_node(cfg, g * cfg.dp_size + team.lane);
      const uint32_t members = __ballot_sync(0xffffffffu, member);
      if (member) {
        s_pend[team.in_block][npend + __popc(members & ((1u << team.lane) - 1u))] =
            tok_arrive_ptr(cfg, st.sync[g * cfg.dp_size + team.lane], t);
      }
      if (team.lane == 0) s_npend[team.in_block] = npend + __popc(members);
      __syncwarp();
      if (npend + 2 * cfg.dp_size > kMaxPending || npend + cfg.dp_size >= 8u * cfg.dp_size) flush();
    }
  };

  // A row whose origin group has members outside the NVLink domain is also copied into the
  // staging buffer, densely inside the group's segment, and its combine slot is written where
  // the proxy reads it. Called by the whole team; returns nullptr when no copy is needed.
  __shared__ uint32_t s_stage_pos[kMaxTeams];
  const bool remote = has_remote(cfg);
  auto stage_row = [&](uint32_t g, uint32_t slot) -> uint8_t* {
    if (!remote) return nullptr;
    bool any = false;
    for (int m = 0; m < cfg.dp_size; ++m) any |= !in_node(cfg, g * cfg.dp_size + m);
    if (!any) return nullptr;   // uniform across the team
    if (team.lane == 0) {
      const uint32_t first = reinterpret_cast<volatile uint32_t*>(ws.proxy)[kProxyRowBase + g];
      const uint32_t pos = first + atom_relaxed_gpu_add(&ws.stage_cursor[g], 1u);
      s_stage_pos[team.in_block] = pos;
      if (pos < cfg.max_recv_rows) reinterpret_cast<volatile uint32_t*>(ws.stage_slot)[pos] = slot;
    }
    team.sync();
    const uint32_t pos = s_stage_pos[team.in_block];
    return pos < cfg.max_recv_rows ? ws.stage + static_cast<uint64_t>(pos) * cfg.c_stride : nullptr;
  };

  if constexpr (WIRE == kWireLL) {
    if (healthy) {
      combine_send_rows_ll<Y>(cfg, st, a, tag_c, meta_rows, meta_recs, TEAM, s_rows, s_wbits, s_n);
    }
  } else if (healthy && cfg.combine_mode == kCombinePerRoute) {
    const uint32_t rows = meta_rows;
    const uint32_t nvec = cfg.c_stride / 16;
    constexpr int U = kCopyUnroll;
    for (uint32_t row = team.id; row < rows; row += team.count) {
      const uint8_t* src = a.expert_y + static_cast<uint64_t>(row) * a.expert_y_stride;
      // the row's bytes do not depend on where it goes: fetch them with its destination
      Vec16 v[U];
      #pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t i = team.lane + u * TEAM;
        if (i < nvec) v[u] = ld_input_v4(src + 16ull * i);
      }
      const uint32_t g = ws.row_src[row];
      const uint32_t tk = ws.row_tk[row];
      if (g == kNoSlot) continue;  // padding row; uniform across the team
      uint8_t* dst[kMaxRanks + 1];
      #pragma unroll
      for (int m = 0; m < kMaxRanks; ++m) {
        dst[m] = (m < cfg.dp_size && in_node(cfg, g * cfg.dp_size + m))
                     ? st.recv[g * cfg.dp_size + m] + cfg.off_crecv + static_cast<uint64_t>(tk) * cfg.c_stride
                     : nullptr;
      }
      dst[kMaxRanks] = stage_row(g, tk);
      for (uint32_t i0 = team.lane; i0 < nvec; i0 += TEAM * U) {
        if (i0 != static_cast<uint32_t>(team.lane)) {
          #pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * TEAM;
            if (i < nvec) v[u] = ld_input_v4(src + 16ull * i);
          }
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t i = i0 + u * TEAM;
          if (i < nvec) {
            #pragma unroll
            for (int m = 0; m <= kMaxRanks; ++m) {
              if (dst[m] != nullptr) st_stream_v4(dst[m] + 16ull * i, v[u]);
            }
          }
        }
      }
      if (row == 0) trace_mark(cfg, ws, kTraceCSendStored);
      team.sync();
      announce(g, tk / K);
      if (row == 0) trace_mark(cfg, ws, kTraceCSendPublished);
    }
    flush();
  } else if (healthy) {
    const uint32_t recs = meta_recs;
    const uint32_t ngran = cfg.hidden_dim / 8;
    for (uint32_t r = team.id; r < recs; r += team.count) {
      const uint32_t t = ws.rec_token[2 * r];
      const uint32_t g = ws.rec_token[2 * r + 1];
      if (team.lane < 32) {
        const int k = team.lane;
        uint32_t row = kNoSlot, wb = 0;
        if (k < K) {
          row = ws.rec_rows[static_cast<uint64_t>(r) * K + k];
          wb = __float_as_uint(ws.rec_weights[static_cast<uint64_t>(r) * K + k]);
        }
        compact_warp(row != kNoSlot, row, wb, s_rows[team.in_block], s_wbits[team.in_block],
                     &s_n[team.in_block]);
      }
      team.sync();
      const uint32_t n = s_n[team.in_block];
      // A record always yields a partial (zeros if none of its rows fitted): the origin counts
      // one arrival per rank it sent the token to.
      const uint64_t slot = static_cast<uint64_t>(t) * cfg.world + st.rank;
      uint8_t* staged = stage_row(g, static_cast<uint32_t>(slot));
      constexpr int GB = 4;  // granules a thread carries at once: GB independent loads per row
      for (uint32_t i0 = team.lane; i0 < ngran; i0 += TEAM * GB) {
        float acc[GB][8];
        #pragma unroll
        for (int u = 0; u < GB; ++u) {
          #pragma unroll
          for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
        }
        for (uint32_t j = 0; j < n; ++j) {
          const uint8_t* row = a.expert_y + static_cast<uint64_t>(s_rows[team.in_block][j]) * a.expert_y_stride;
          const float w = __uint_as_float(s_wbits[team.in_block][j]);
          float f[GB][8];
          #pragma unroll
          for (int u = 0; u < GB; ++u) {
            const uint32_t i = i0 + u * TEAM;
            if (i < ngran) Elem8<Y>::load(row + static_cast<uint64_t>(i) * Elem8<Y>::kBytes, f[u], false);
          }
          #pragma unroll
          for (int u = 0; u < GB; ++u) {
            const uint32_t i = i0 + u * TEAM;
            if (i < ngran) {
              #pragma unroll
              for (int q = 0; q < 8; ++q) acc[u][q] = fmaf(w, f[u][q], acc[u][q]);
            }
          }
        }
        #pragma unroll
        for (int u = 0; u < GB; ++u) {
          const uint32_t i = i0 + u * TEAM;
          if (i < ngran) {
              for (int m = 0; m < cfg.dp_size; ++m) {
                if (!in_node(cfg, g * cfg.dp_size + m)) continue;
                Elem8<Y>::store(st.recv[g * cfg.dp_size + m] + cfg.off_crecv + slot * cfg.c_stride +
                                    static_cast<uint64_t>(i) * Elem8<Y>::kBytes,
                                acc[u]);
              }
              if (staged != nullptr) {
                Elem8<Y>::store(staged + static_cast<uint64_t>(i) * Elem8<Y>::kBytes, acc[u]);
              }
          }
        }
      }
      team.sync();
      announce(g, t);
    }
    flush();
  }
  proxy_phase_done(cfg, ws, 1, tag_c);
  trace_mark(cfg, ws, kTraceCSendLoopDone);
  trace_max(cfg, ws, kTraceCSendLoopLast);
}

// ---------------------------------------------------------------------------
// combine_recv
// ---------------------------------------------------------------------------

template <int WIRE, typename Y, typename O>
__device__ void combine_recv_phase(const A2AConfig& cfg, const A2ARankState& st,
                                   const CombineRecvArgs& a, const int TEAM) {
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  const uint32_t epoch = read_epoch(ws, 1);
  trace_mark(cfg, ws, kTraceCRecvStart);

  __shared__ uint32_t s_abort;
  __shared__ uint32_t s_slot[kMaxTeams][kMaxTopK];
  __shared__ uint32_t s_wbits[kMaxTeams][kMaxTopK];
  __shared__ uint32_t s_n[kMaxTeams];

  int T = a.num_tokens;
  if (a.bound_m != nullptr) T = min(T, *a.bound_m);
  T = max(0, min(T, cfg.max_num_tokens));

  if (threadIdx.x == 0) s_abort = ws.status[0] != 0 ? 1u : 0u;
  __syncthreads();
  if (has_remote(cfg)) {
    // rows from ranks outside the NVLink domain come through the transfer engine; their proxy
    // announces them all at once, after the last one has landed
    if (threadIdx.x < cfg.world && !in_node(cfg, threadIdx.x)) {
      uint64_t waited;
      const bool ok = wait_flag(flag_ptr(st.sync[st.rank], kFlagRemoteCombine, threadIdx.x), epoch + 1,
                                cfg.wait_limit_ns, &waited);
      if (!ok) {
        report(ws, kStatusWaitTimeout, kPhaseCombineRecv, threadIdx.x, epoch + 1);
        s_abort = 1;
      }
    }
    __syncthreads();
  }
  if (a.external) {
    // the sending kernels announce a whole rank's rows at once
    const uint32_t expected = read_epoch(ws, 2) + 1;
    if (threadIdx.x < cfg.world) {
      uint64_t waited;
      const bool ok = wait_flag(flag_ptr(st.sync[st.rank], kFlagExternalCombine, threadIdx.x),
                                expected, cfg.wait_limit_ns, &waited);
      if (!ok) {
        report(ws, kStatusWaitTimeout, kPhaseCombineRecv, threadIdx.x, expected);
        s_abort = 1;
      }
      if (blockIdx.x == 0) atomicMax(&ws.stats[3], static_cast<unsigned long long>(waited));
    }
    __syncthreads();
  }
  trace_mark(cfg, ws, kTraceCRecvWaitDone);

  if constexpr (WIRE == kWireLL) {
    if (s_abort == 0) combine_recv_tokens_ll<Y, O>(cfg, st, a, T, epoch + 1, TEAM, s_slot, s_wbits, s_n);
  } else if (s_abort == 0) {
    const uint8_t* crecv = st.recv[st.rank] + cfg.off_crecv;
    const uint32_t ngran = cfg.hidden_dim / 8;
    for (int t = team.id; t < T; t += team.count) {
      if (team.lane < 32) {
        combine_sources(cfg, a, t, s_slot[team.in_block], s_wbits[team.in_block],
                        &s_n[team.in_block]);
        __syncwarp();
        const uint32_t n_local = has_remote(cfg) ? combine_local_sources(cfg, a, t) : s_n[team.in_block];
        if (team.lane == 0 && !a.external) {
          const uint32_t n = n_local;
          uint32_t* counter = tok_arrive_ptr(cfg, st.sync[st.rank], static_cast<uint32_t>(t));
          if (n != 0) {
            if (wait_word(counter, n, false, cfg.wait_limit_ns, ws.status)) {
              // the next rows for this token come after this rank's next dispatch
              *reinterpret_cast<volatile uint32_t*>(counter) = 0;
            } else {
              report(ws, kStatusWaitTimeout, kPhaseCombineRecv, t, n);
              s_n[team.in_block] = kTeamAbort;
            }
          }
        }
      }
      team.sync();
      if (t == 0) trace_mark(cfg, ws, kTraceCRecvFirstToken);
      const uint32_t n = s_n[team.in_block];
      if (n == kTeamAbort) break;  // uniform across the team
      uint8_t* out_row = a.out_tokens + static_cast<uint64_t>(t) * a.out_tokens_stride * sizeof(O);
      for (uint32_t i = team.lane; i < ngran; i += TEAM) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (a.accumulate) {
          Elem8<O>::load(out_row + static_cast<uint64_t>(i) * Elem8<O>::kBytes, acc, true);
        }
        weighted_gather8<Y>(acc, crecv, cfg.c_stride, s_slot[team.in_block],
                            s_wbits[team.in_block], n, static_cast<uint64_t>(i) * Elem8<Y>::kBytes,
                            true);
        Elem8<O>::store(out_row + static_cast<uint64_t>(i) * Elem8<O>::kBytes, acc);
      }
      team.sync();
    }
  }
  trace_mark(cfg, ws, kTraceCRecvLoopDone);
  trace_max(cfg, ws, kTraceCRecvLoopLast);
  finish_recv(cfg, ws, 1, epoch, kTraceCRecvAllDone, a.external != 0);
}

// ---------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------

template <int WIRE>
__global__ void __launch_bounds__(kA2AThreads, 1)
dispatch_kernel(const __grid_constant__ A2AConfig cfg, const __grid_constant__ A2ARankStates states,
                const __grid_constant__ PerRank<DispatchSendArgs> send,
                const __grid_constant__ PerRank<DispatchRecvArgs> recv, int send_team,
                int recv_team) {
  extern __shared__ __align__(16) uint32_t dyn_smem[];
  const A2ARankState& st = states.r[blockIdx.y];
  if (send_team) dispatch_send_phase<WIRE>(cfg, st, send.r[blockIdx.y], dyn_smem, send_team);
  if (send_team && recv_team) __syncthreads();
  if (recv_team) dispatch_recv_phase<WIRE>(cfg, st, recv.r[blockIdx.y], dyn_smem, recv_team);
}

template <int WIRE, typename Y>
__global__ void __launch_bounds__(kA2AThreads, 1)
combine_send_kernel(const __grid_constant__ A2AConfig cfg,
                    const __grid_constant__ A2ARankStates states,
                    const __grid_constant__ PerRank<CombineSendArgs> send, int send_team) {
  combine_send_phase<WIRE, Y>(cfg, states.r[blockIdx.y], send.r[blockIdx.y], send_team);
}

template <int WIRE, typename Y, typename O>
__global__ void __launch_bounds__(kA2AThreads, 1)
combine_recv_kernel(const __grid_constant__ A2AConfig cfg,
                    const __grid_constant__ A2ARankStates states,
                    const __grid_constant__ PerRank<CombineRecvArgs> recv, int recv_team) {
  combine_recv_phase<WIRE, Y, O>(cfg, states.r[blockIdx.y], recv.r[blockIdx.y], recv_team);
}

template <int WIRE, typename Y, typename O>
__global__ void __launch_bounds__(kA2AThreads, 1)
combine_kernel(const __grid_constant__ A2AConfig cfg, const __grid_constant__ A2ARankStates states,
               const __grid_constant__ PerRank<CombineSendArgs> send,
               const __grid_constant__ PerRank<CombineRecvArgs> recv, int send_team,
               int recv_team) {
  combine_send_phase<WIRE, Y>(cfg, states.r[blockIdx.y], send.r[blockIdx.y], send_team);
  __syncthreads();
  combine_recv_phase<WIRE, Y, O>(cfg, states.r[blockIdx.y], recv.r[blockIdx.y], recv_team);
}

// Every rank announces itself on every rank's barrier counters and waits until it has heard
// from all of them. One block per rank; used to line ranks up (benchmarks, tests, teardown),
// never inside dispatch or combine.
__global__ void __launch_bounds__(32, 1)
barrier_kernel(const __grid_constant__ A2AConfig cfg, const __grid_constant__ A2ARankStates states) {
  const A2ARankState& st = states.r[blockIdx.y];
  const A2ALocal& ws = st.local;
  const uint32_t expected = read_epoch(ws, 3) + 1;
  __syncwarp();
  if (threadIdx.x < cfg.world && in_node(cfg, threadIdx.x)) {   // the NVLink domain only
    red_release_sys_add(flag_ptr(st.sync[threadIdx.x], kFlagBarrier, st.rank), 1u);
    uint64_t waited;
    if (!wait_flag(flag_ptr(st.sync[st.rank], kFlagBarrier, threadIdx.x), expected,
                   cfg.wait_limit_ns, &waited)) {
      report(ws, kStatusWaitTimeout, kNumPhases, threadIdx.x, expected);
    }
  }
  __syncwarp();
  if (threadIdx.x == 0) ws.epochs[3] = expected;
}

size_t dispatch_smem_bytes(const A2AConfig& cfg, int send_team, int recv_team, bool quantize) {
  size_t bytes = dispatch_stage_offset(cfg);
  if (cfg.wire == kWireLL) {
    size_t side = 0;
    if (send_team > 0) side = (kA2AThreads / send_team) * ll_side_bytes(cfg, quantize);
    if (recv_team > 0) side = std::max(side, (kA2AThreads / recv_team) * ll_side_bytes(cfg, false));
    bytes += side;
  }
  return bytes;
}

template <typename F>
cudaError_t with_dtype(int dtype, F&& f) {
  switch (dtype) {
    case kDtypeBF16: return f(static_cast<__nv_bfloat16*>(nullptr));
    case kDtypeF16: return f(static_cast<__half*>(nullptr));
    case kDtypeF32: return f(static_cast<float*>(nullptr));
    default: return cudaErrorInvalidValue;
  }
}

template <typename Kern, typename... Args>
cudaError_t launch(Kern kern, dim3 grid, size_t smem, cudaStream_t stream, bool cooperative,
                   Args... args) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  void* params[] = {const_cast<void*>(static_cast<const void*>(&args))...};
  if (cooperative) {
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), grid,
                                       dim3(kA2AThreads), params, smem, stream);
  }
  return cudaLaunchKernel(reinterpret_cast<const void*>(kern), grid, dim3(kA2AThreads), params,
                          smem, stream);
}

}  // namespace

int a2a_pick_team(const A2AConfig& cfg, int64_t work_items, int64_t vectors_per_item) {
  // A team handles its items one after the other and each item in batches of
  // TEAM x kCopyUnroll vectors; both are latency-bound round trips. Pick the team size
  // with the fewest sequential round trips (ties go to the wider team).
  const int64_t warps = static_cast<int64_t>(cfg.num_blocks) * (kA2AThreads / 32);
  int best_team = 512;
  int64_t best_cost = INT64_MAX;
  for (int team : {512, 128, 32}) {
    const int64_t teams = warps / (team / 32);
    const int64_t rounds = (work_items + teams - 1) / teams;
    const int64_t per_batch = static_cast<int64_t>(team) * kCopyUnroll;
    const int64_t batches = (vectors_per_item + per_batch - 1) / per_batch;
    const int64_t cost = rounds * batches;
    if (cost < best_cost) {
      best_cost = cost;
      best_team = team;
    }
  }
  return best_team;
}

cudaError_t a2a_launch_dispatch(const A2AConfig& cfg, const A2ARankStates& states, int nranks,
                                const PerRank<DispatchSendArgs>& send,
                                const PerRank<DispatchRecvArgs>& recv, int send_team, int recv_team,
                                cudaStream_t stream) {
  const dim3 grid(cfg.num_blocks, nranks);
  bool quantize = false;
  for (int i = 0; i < nranks; ++i) quantize |= send_team && send.r[i].quantize != 0;
  const size_t smem = dispatch_smem_bytes(cfg, send_team, recv_team, quantize);
  // One launch that plays several ranks contains blocks that wait for one another:
  // co-residency must be guaranteed (or the launch refused) by the driver.
  const bool cooperative = nranks > 1 && send_team && recv_team;
  if (cfg.wire == kWireLL) {
    return launch(dispatch_kernel<kWireLL>, grid, smem, stream, cooperative, cfg, states, send, recv,
                  send_team, recv_team);
  }
  return launch(dispatch_kernel<kWirePlain>, grid, smem, stream, cooperative, cfg, states, send, recv,
                send_team, recv_team);
}

namespace {
template <int WIRE>
cudaError_t preload_wire() {
  cudaFuncAttributes attr;
  cudaError_t e = cudaFuncGetAttributes(&attr, dispatch_kernel<WIRE>);
  if (e != cudaSuccess) return e;
  const int dtypes[] = {kDtypeBF16, kDtypeF16, kDtypeF32};
  for (int y : dtypes) {
    e = with_dtype(y, [&](auto* yp) {
      using Y = std::remove_pointer_t<decltype(yp)>;
      cudaError_t r = cudaFuncGetAttributes(&attr, combine_send_kernel<WIRE, Y>);
      for (int o : dtypes) {
        if (r != cudaSuccess) break;
        r = with_dtype(o, [&](auto* op) {
          using O = std::remove_pointer_t<decltype(op)>;
          cudaError_t q = cudaFuncGetAttributes(&attr, combine_kernel<WIRE, Y, O>);
          if (q == cudaSuccess) q = cudaFuncGetAttributes(&attr, combine_recv_kernel<WIRE, Y, O>);
          return q;
        });
      }
      return r;
    });
    if (e != cudaSuccess) return e;
  }
  return cudaFuncGetAttributes(&attr, barrier_kernel);
}
}  // namespace

cudaError_t a2a_preload_kernels(const A2AConfig& cfg) {
  return cfg.wire == kWireLL ? preload_wire<kWireLL>() : preload_wire<kWirePlain>();
}

cudaError_t a2a_launch_barrier(const A2AConfig& cfg, const A2ARankStates& states, int nranks,
                               cudaStream_t stream) {
  void* params[] = {const_cast<void*>(static_cast<const void*>(&cfg)),
                    const_cast<void*>(static_cast<const void*>(&states))};
  const dim3 grid(1, nranks);
  if (nranks > 1) {
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(barrier_kernel), grid, dim3(32),
                                       params, 0, stream);
  }
  return cudaLaunchKernel(reinterpret_cast<const void*>(barrier_kernel), grid, dim3(32), params, 0,
                          stream);
}

template <int WIRE>
cudaError_t launch_combine_wire(const A2AConfig& cfg, const A2ARankStates& states, int nranks,
                                const PerRank<CombineSendArgs>& send,
                                const PerRank<CombineRecvArgs>& recv, int send_team, int recv_team,
                                int y_dtype, int out_dtype, cudaStream_t stream) {
  const dim3 grid(cfg.num_blocks, nranks);
  return with_dtype(y_dtype, [&](auto* yp) {
    using Y = std::remove_pointer_t<decltype(yp)>;
    if (send_team && !recv_team) {
      return launch(combine_send_kernel<WIRE, Y>, grid, 0, stream, false, cfg, states, send, send_team);
    }
    return with_dtype(out_dtype, [&](auto* op) {
      using O = std::remove_pointer_t<decltype(op)>;
      if (send_team) {
        return launch(combine_kernel<WIRE, Y, O>, grid, 0, stream, nranks > 1, cfg, states, send, recv,
                      send_team, recv_team);
      }
      return launch(combine_recv_kernel<WIRE, Y, O>, grid, 0, stream, false, cfg, states, recv, recv_team);
    });
  });
}

cudaError_t a2a_launch_combine(const A2AConfig& cfg, const A2ARankStates& states, int nranks,
                               const PerRank<CombineSendArgs>& send,
                               const PerRank<CombineRecvArgs>& recv, int send_team, int recv_team,
                               int y_dtype, int out_dtype, cudaStream_t stream) {
  if (cfg.wire == kWireLL) {
    return launch_combine_wire<kWireLL>(cfg, states, nranks, send, recv, send_team, recv_team, y_dtype,
                                        out_dtype, stream);
  }
  return launch_combine_wire<kWirePlain>(cfg, states, nranks, send, recv, send_team, recv_team, y_dtype,
                                         out_dtype, stream);
}

}  // namespace pplx

