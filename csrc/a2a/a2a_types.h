// Plain-data description of one expert-parallel all-to-all context.
//
// The protocol is device-only: every rank owns a *symmetric* region (same layout
// on every rank, mapped into every peer over NVLink) made of
//
//   flags    one 128-byte line per (kind, source rank): "dispatch n has started here"
//            words, arrival counters of externally sent combines, barrier counters
//   counts   two banks (dispatch parity) x source dp-group: {#records for this rank,
//            per-local-expert token counts}
//   tokens   one arrival counter per local token: combine rows that have landed
//   drecv    dispatch records, one fixed-capacity region per source dp-group
//   crecv    combine records, indexed by the origin's (token, k) or (token, rank)
//
// A dispatch record is sent once per (token, destination rank) and replicated to
// the experts of that rank on arrival:
//
//   [ header | payload (hidden * in_elemsize, 16-byte padded) | scales ]
//   header words: [0] epoch tag (dispatch number + 1), [1] source token, [2..2+K) expert
//   ids, [2+K..2+2K) fp32 routing weights; padded to 16 bytes.
// The sender packs the records for one destination densely (slot = an atomic cursor per
// destination) and tells the destination how many there are in the counts message, which
// leaves before any payload. The tag is the last word of a record to be written, with
// release semantics: a receiver that sees the current tag in a slot may read that record
// at once, without waiting for any other (regions are zero-filled once, tags start at 1).
// A combine row is announced the same way, by a release-scoped increment of the arrival
// counter of its token at the origin, so token t is reduced as soon as its rows are in.
//
// The reference sends one copy per route and keeps a 16-byte reserved trailer
// instead (p2p-all-to-all/a2a-kernels/src/a2a/a2a_dispatch_send.cu:586-588,
// p2p-all-to-all/src/a2a_worker.rs:317-325).
#pragma once

#include <cstddef>
#include <cstdint>

namespace pplx {

constexpr int kMaxRanks = 8;          // one NVSwitch domain
constexpr int kMaxTopK = 16;
constexpr int kMaxVirtualRanks = 8;   // ranks emulated by one launch on one GPU
constexpr int kA2AThreads = 512;
constexpr uint32_t kNoSlot = 0xffffffffu;
constexpr int kFlagStrideWords = 32;  // 128 bytes per flag

enum A2APhase : int {
  kPhaseDispatchSend = 0,
  kPhaseDispatchRecv = 1,
  kPhaseCombineSend = 2,
  kPhaseCombineRecv = 3,
  kNumPhases = 4,
};

// Slots of the optional timeline (globaltimer ns, written by block 0 / the last block).
enum A2ATrace : int {
  kTraceSendStart = 0, kTraceSendLoopDone = 1, kTraceSendSignalled = 2,
  kTraceRecvStart = 3, kTraceRecvWaitDone = 4, kTraceRecvLayoutDone = 5,
  kTraceRecvLoopDone = 6, kTraceRecvAllDone = 7,
  kTraceCSendStart = 8, kTraceCSendLoopDone = 9, kTraceCSendSignalled = 10,
  kTraceCRecvStart = 11, kTraceCRecvWaitDone = 12, kTraceCRecvLoopDone = 13,
  kTraceCRecvAllDone = 14,
  // finer points, block 0 / first item unless stated otherwise
  kTraceSendSlots = 15,        // record slots of the first token allocated
  kTraceSendStored = 16,       // its stores issued
  kTraceSendPublished = 17,    // its tag released
  kTraceRecvFirstTag = 18,     // first record's tag seen
  kTraceSendLoopLast = 19,     // latest block to leave the send loop
  kTraceRecvLoopLast = 20,     // latest block to leave the record loop
  kTraceCSendStored = 21,      // first row's stores issued
  kTraceCSendPublished = 22,   // first row announced
  kTraceCRecvFirstToken = 23,  // first token's rows all in
  kTraceCSendLoopLast = 24,    // latest block to leave the combine send loop
  kTraceCRecvLoopLast = 25,    // latest block to leave the reduction loop
  kTraceSlots = 32,
};

// Rows of the flag table at the start of the sync region (one 128-byte line per source rank).
enum A2AFlagRow : int {
  kFlagDispatchStarted = 0,  // tag of the newest dispatch whose counts message rank s sent here
  kFlagExternalCombine = 1,  // combines whose send phase another kernel of rank s played
  kFlagBarrier = 2,          // barriers rank s has entered
  kFlagRemoteCombine = 3,    // tag of the newest combine whose rows rank s (a rank outside this
                             // NVLink domain) has delivered here through the transfer engine
  kNumFlagRows = 4,
};

// Words of the pinned host block through which the kernels talk to the host proxy that serves
// ranks outside the NVLink domain (A2ALocal::proxy).
enum A2AProxyWord : int {
  kProxyDispatchSent = 0,   // tag of the newest dispatch whose send phase has finished on this rank
  kProxyCombineSent = 1,    // same for the combine
  kProxyRecords = 8,        // [kMaxRanks] records staged for each destination rank by that dispatch
  kProxyRows = 16,          // [kMaxRanks] rows staged for each origin dp group by that combine
  kProxyRowBase = 24,       // [kMaxRanks] first staged row of each origin dp group
  kProxyWords = 32,
};

// Values of status[0]. status[1] = phase, status[2] = peer/group, status[3] = detail.
enum A2AStatus : uint32_t {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,     // a bounded wait on an arrival flag ran out
  kStatusRowOverflow = 2,     // more expert rows than the output tensor holds
  kStatusBadExpertIndex = 3,  // indices[t][k] >= num_experts
  kStatusRecordOverflow = 4,  // more records than a source region holds
  kStatusBadRecord = 5,       // a record header names a token or count outside its limits
};

enum A2AWire : int {
  kWireAuto = 0,
  kWirePlain = 1,  // contiguous records; arrival announced by release stores / counters
  kWireLL = 2,     // 128-byte lines of 112 data bytes + a 16-byte flag vector (see a2a_ll.cuh)
};

enum A2ACombineMode : int {
  kCombinePerRoute = 0,   // one record per (token, k); weights applied at the origin
  kCombinePreReduce = 1,  // expert rank applies the dispatch-time weights and sends
                          // one partial sum per (token, expert rank)
};

struct A2AConfig {
  int world;             // ranks in the NVLink domain
  int dp_size;           // ranks that hold identical tokens (TP replication factor)
  int num_groups;        // world / dp_size
  int num_experts;
  int experts_per_rank;  // ceil(num_experts / world)
  int topk;
  int max_num_tokens;    // per dp group and per call
  int hidden_dim;
  int hidden_dim_scale;  // 0 when there are no scales
  int in_elemsize;
  int out_elemsize;      // element size of combine records (expert_y)
  int expert_padding;
  int combine_mode;
  int num_blocks;        // grid.x of every a2a kernel (arrival counters depend on it)
  int trace;             // 1: kernels record a coarse timeline into A2ALocal::trace
  int wire;              // A2AWire, never kWireAuto here
  uint32_t node_mask;    // bit r: rank r is in this rank's NVLink domain (its memory is mapped
                         // here); the other ranks are served by the host proxy

  // wire format
  uint32_t d_header_bytes;
  uint32_t d_payload_bytes;
  uint32_t d_scale_bytes;
  uint32_t d_stride;       // bytes per dispatch record
  uint32_t c_stride;       // bytes per combine record
  uint32_t c_records_per_token;  // topk (per-route) or world (pre-reduce)
  uint32_t counts_stride;  // u32 words per source group in the counts table
  uint32_t max_recv_rows;  // capacity of the row tables (expert-major rows)

  // symmetric layout, byte offsets
  uint64_t sync_bytes;
  uint64_t off_counts;          // inside the sync region; two banks of counts_bank_words
  uint64_t off_tok_arrive;      // inside the sync region; [max_num_tokens] u32
  uint32_t counts_bank_words;   // counts_stride x the number of senders of a counts message: the source
                                // groups, or every source rank in the flagged-line format
  uint32_t pad0_;
  uint64_t recv_bytes;
  uint64_t off_drecv;           // inside the recv region
  uint64_t drecv_group_stride;
  uint64_t off_crecv;

  uint64_t wait_limit_ns;
};

// Device-local (not peer visible) workspace of one rank.
struct A2ALocal {
  uint32_t* epochs;        // [0] completed dispatches, [1] completed combines, [2] of those the
                           // ones whose send was external; advanced by the last block of the
                           // respective *recv* phase. [3] barriers entered.
  uint32_t* done;          // [2] blocks that finished the current recv phase
  uint32_t* send_cursor;   // [2][kMaxRanks] next free record slot per destination, by parity
  uint32_t* place_cursor;  // [2][num_groups * experts_per_rank], indexed by epoch parity
  uint32_t* row_src;       // [max_recv_rows] source dp group of a row, kNoSlot = padding
  uint32_t* row_tk;        // [max_recv_rows] token * topk + k at the source
  uint32_t* expert_meta;   // [0] padded row count, [1] record count,
                           // [2 .. 2+L) totals, [2+L .. 2+2L) padded offsets
  uint32_t* rec_rows;      // pre-reduce: [num_groups * max_num_tokens][topk] row or kNoSlot
  float* rec_weights;      // pre-reduce: same shape, routing weight
  uint32_t* rec_token;     // pre-reduce: [num_groups * max_num_tokens] token index
  uint32_t* status;        // [4]
  uint32_t* host_flag;     // pinned host word (device-mapped): failure code, readable by the
                           // host without synchronising the stream
  // ---- routing fused into the dispatch: counts gathered from all blocks ----
  uint32_t* route_hist;    // [2][num_experts] routes per expert, by dispatch parity
  uint32_t* route_nrec;    // [2][kMaxRanks] records per destination rank
  uint32_t* route_done;    // [2] blocks that have routed all their tokens
  // ---- only used when some rank is outside the NVLink domain ----
  uint32_t* proxy;         // pinned host words (device-mapped), see A2AProxyWord
  uint32_t* send_done;     // [2] blocks that finished the current dispatch / combine send phase
  uint8_t* stage;          // [max_recv_rows] combine rows bound for ranks outside the domain
  uint32_t* stage_slot;    // pinned host (device-mapped): [max_recv_rows] combine slot of each staged row
  uint32_t* stage_cursor;  // [kMaxRanks] rows staged so far for each origin dp group
  unsigned long long* stats;  // [8] counters: tokens sent, -, max dispatch/combine wait ns
  unsigned long long* trace;  // [kTraceSlots] see A2ATrace
};

struct A2ARankState {
  int rank;
  int pad_;
  A2ALocal local;
  uint8_t* sync[kMaxRanks];  // every rank's sync region as mapped here
  uint8_t* recv[kMaxRanks];  // every rank's recv region as mapped here
};

struct A2ARankStates {
  A2ARankState r[kMaxVirtualRanks];
};

struct DispatchSendArgs {
  const uint8_t* x;
  uint64_t x_stride;  // bytes
  const uint8_t* x_scale;
  int64_t x_scale_stride_elem;   // in elements
  int64_t x_scale_stride_token;  // in elements
  const uint32_t* indices;
  uint64_t indices_stride;  // elements
  const float* weights;
  uint64_t weights_stride;  // elements
  const int32_t* bound_m;
  int32_t num_tokens;
  int32_t quantize;  // 1: x is bf16 and is quantised to e4m3 with 1x128 scales on the fly; 2: the same with
                     // scales rounded up to powers of two
  // Routing fused into the dispatch: when `logits` is set, the team that sends a token first picks
  // its top-k experts (on logit + bias) and the softmax weights over the chosen logits, writes
  // them to `indices` / `weights` (outputs then, the combine reads them later) and sends by them.
  const void* logits;          // [num_tokens, num_experts] fp32 or bf16, nullptr: routing is given
  int64_t logits_stride;       // elements
  const float* logits_bias;    // [num_experts] or nullptr
  int32_t logits_bf16;
  int32_t pad_;
};

struct DispatchRecvArgs {
  int32_t* out_num_tokens;
  uint8_t* out_x;
  uint64_t out_x_stride;  // bytes
  uint8_t* out_x_scale;
  int64_t out_x_scale_stride_elem;
  int64_t out_x_scale_stride_token;
  uint32_t out_rows;  // rows available in out_x (0 = unknown: trust max_recv_rows)
  uint32_t pad_;
};

struct CombineSendArgs {
  const uint8_t* expert_y;
  uint64_t expert_y_stride;  // bytes
};

struct CombineRecvArgs {
  uint8_t* out_tokens;
  uint64_t out_tokens_stride;  // elements
  const uint32_t* indices;
  uint64_t indices_stride;
  const float* weights;
  uint64_t weights_stride;
  const int32_t* bound_m;
  int32_t num_tokens;
  int32_t accumulate;
  int32_t external;  // 1: the rows were written by another kernel, which announced them per
                     // source rank (kFlagExternalCombine) instead of per token
  int32_t pad_;
};

template <typename T>
struct PerRank {
  T r[kMaxVirtualRanks];
};

// Scalar types understood by the combine kernel (values match torch's ScalarType).
enum A2ADtype : int {
  kDtypeF16 = 5,
  kDtypeF32 = 6,
  kDtypeBF16 = 15,
};

static inline uint64_t round_up_u64(uint64_t a, uint64_t b) { return (a + b - 1) / b * b; }

}  // namespace pplx
