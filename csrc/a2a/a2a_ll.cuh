// Flag-in-line wire format ("LL") for latency-bound sizes.
//
// A record or row is cut into 128-byte lines of seven 16-byte data vectors plus one flag
// vector that repeats the epoch tag. A line is stored by eight neighbouring lanes of one warp
// in one instruction and read back the same way, so it travels and is observed as one unit:
// a reader that finds the current tag in the flag vector of a line has that line's data.
// No fence, no separate arrival signal and no wait for anything but the line itself: the
// sender never stalls on the drain of its stores and the receiver consumes data in the order
// in which it lands. The cost is one eighth more bytes on the wire, so contexts built for
// many tokens per call keep the plain format, whose arrival signals are release stores.
//
// The reference moves payload and flags separately and orders them with a system-scope
// release after a grid barrier (p2p-all-to-all/a2a-kernels/src/a2a/a2a_dispatch_send.cu:525-535).
#pragma once

#include "a2a_device.cuh"

namespace pplx {
namespace {

__device__ __forceinline__ bool ll_is_flag(uint32_t p) { return (p & 7u) == 7u; }
__device__ __forceinline__ uint32_t ll_logical(uint32_t p) { return (p >> 3) * 7u + (p & 7u); }

__device__ __forceinline__ Vec16 ld_volatile_v4(const void* p) {
  Vec16 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Warp-collective: every lane loads up to U physical vectors, the u-th from addr(u), and the
// call returns once every line touched carries `tag` (true) or the wait ran out (false).
// Lanes of one aligned group of eight must address the eight vectors of one line for the same
// u; `active(u)` must be uniform across such a group. A lane's v[u] is only meaningful where
// active(u) held.
template <int U, typename Addr, typename Active>
__device__ __forceinline__ bool ll_load_lines(Vec16 (&v)[U], uint32_t tag, Addr addr, Active active,
                                              uint64_t limit_ns, const uint32_t* status) {
  const uint32_t flag_lane = (threadIdx.x & 24u) | 7u;
  uint32_t pending = 0;
  #pragma unroll
  for (int u = 0; u < U; ++u) pending |= active(u) ? (1u << u) : 0u;
  uint64_t start = 0;
  for (uint32_t spin = 0;; ++spin) {
    #pragma unroll
    for (int u = 0; u < U; ++u) {
      if ((pending >> u) & 1u) v[u] = ld_volatile_v4(addr(u));
    }
    #pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t mine = (v[u].x == tag && v[u].w == tag) ? 1u : 0u;
      const uint32_t ok = __shfl_sync(0xffffffffu, mine, flag_lane);
      if (ok) pending &= ~(1u << u);
    }
    if (__all_sync(0xffffffffu, pending == 0)) return true;
    if ((spin & 63u) == 63u) {
      const uint64_t now = globaltimer_ns();
      if (start == 0) start = now;
      const bool give_up = now - start > limit_ns ||
                           *reinterpret_cast<const volatile uint32_t*>(status) != 0;
      if (__any_sync(0xffffffffu, give_up)) return false;
    }
  }
}

// 16 bytes of Y as floats and back.
template <typename Y>
struct VecElems;

template <>
struct VecElems<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void unpack(const Vec16& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  __device__ static __forceinline__ void pack(const float* f, uint32_t* out) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(out);
    #pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};

template <>
struct VecElems<__half> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void unpack(const Vec16& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __half22float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  __device__ static __forceinline__ void pack(const float* f, uint32_t* out) {
    __half2* h = reinterpret_cast<__half2*>(out);
    #pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
};

template <>
struct VecElems<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void unpack(const Vec16& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ void pack(const float* f, uint32_t* out) {
    #pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = __float_as_uint(f[i]);
  }
};

// N floats written as N elements of O starting at element index `elem` of `row`.
template <typename O, int N>
__device__ __forceinline__ void store_elems(uint8_t* row, uint64_t elem, const float* f) {
  uint32_t w[8];
  if constexpr (sizeof(O) == 4) {
    #pragma unroll
    for (int i = 0; i < N; ++i) w[i] = __float_as_uint(f[i]);
    #pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      st_stream_v4(row + elem * 4 + 16 * i, Vec16{w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]});
    }
  } else {
    if constexpr (N == 8) {
      VecElems<O>::pack(f, w);
      st_stream_v4(row + elem * 2, Vec16{w[0], w[1], w[2], w[3]});
    } else {
      // four elements of a 2-byte type: one 8-byte store
      float g[8] = {f[0], f[1], f[2], f[3], 0.f, 0.f, 0.f, 0.f};
      VecElems<O>::pack(g, w);
      asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};"
                   :
                   : "l"(row + elem * 2), "r"(w[0]), "r"(w[1])
                   : "memory");
    }
  }
}

template <typename O, int N>
__device__ __forceinline__ void load_elems(const uint8_t* row, uint64_t elem, float* f) {
  if constexpr (sizeof(O) == 4) {
    #pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const Vec16 v = ld_stream_v4(row + elem * 4 + 16 * i);
      f[4 * i] = __uint_as_float(v.x); f[4 * i + 1] = __uint_as_float(v.y);
      f[4 * i + 2] = __uint_as_float(v.z); f[4 * i + 3] = __uint_as_float(v.w);
    }
  } else {
    const O* p = reinterpret_cast<const O*>(row) + elem;
    #pragma unroll
    for (int i = 0; i < N; ++i) f[i] = static_cast<float>(p[i]);
  }
}

// Code size matters here: these paths run once per launch on a cold instruction cache, so the
// loops below keep only the loads unrolled (to have several in flight) and leave everything
// else rolled.
// Vectors a lane has in flight per batch: with 128-thread teams one batch covers a DeepSeek-V3
// dispatch record (536 vectors) and one a combine row (1024 vectors).
constexpr int kLLUnrollDispatch = 5;
constexpr int kLLUnrollCombine = 8;

// Per-team scratch in dynamic shared memory: [header | scales | payload (fused quantisation)].
struct LLSide {
  uint32_t* hdr;     // d_header_bytes
  uint8_t* scales;   // d_scale_bytes
  uint8_t* payload;  // d_payload_bytes, only when the launch quantises
};

__host__ __device__ inline size_t ll_side_bytes(const A2AConfig& cfg, bool with_payload) {
  return cfg.d_header_bytes + cfg.d_scale_bytes + (with_payload ? cfg.d_payload_bytes : 0);
}

__device__ __forceinline__ LLSide ll_side(const A2AConfig& cfg, uint8_t* base, int in_block,
                                         bool with_payload) {
  uint8_t* p = base + static_cast<size_t>(in_block) * ll_side_bytes(cfg, with_payload);
  return LLSide{reinterpret_cast<uint32_t*>(p), p + cfg.d_header_bytes,
                p + cfg.d_header_bytes + cfg.d_scale_bytes};
}

// ---------------------------------------------------------------------------
// dispatch, sender side: one team per token, records written as flagged lines
// ---------------------------------------------------------------------------

// Logical layout of a record (16-byte vectors): header | payload | scales, as in the plain
// format; the tag word of the header is filled in too but nobody waits on it.
template <typename Route>
__device__ void dispatch_send_tokens_ll(const A2AConfig& cfg, const A2ARankState& st,
                                        const DispatchSendArgs& a, int T, uint32_t tag, uint32_t par,
                                        const int TEAM, uint8_t* side_base, Route route) {
  const bool fused_route = a.logits != nullptr;
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  const int world = cfg.world;
  const int K = cfg.topk;
  const int L = cfg.experts_per_rank;
  const int my_group = st.rank / cfg.dp_size;
  const int my_tp = st.rank % cfg.dp_size;
  const uint32_t hdr_vecs = cfg.d_header_bytes / 16;
  const uint32_t nvec = cfg.d_payload_bytes / 16;
  const int hs = cfg.hidden_dim_scale;
  const uint32_t scale_vecs = cfg.d_scale_bytes / 16;
  const uint32_t nphys = cfg.d_stride / 16;  // lines * 8
  constexpr int U = kLLUnrollDispatch;
  const bool quant = a.quantize != 0;
  const LLSide side = ll_side(cfg, side_base, team.in_block, quant);
  __shared__ uint8_t* s_dst[kMaxTeams][kMaxRanks];
  __shared__ uint32_t s_ndst[kMaxTeams];
  const Vec16 flag = {tag, tag, tag, tag};

  #pragma unroll 1
  for (int t = team.id; t < T; t += team.count) {
    const uint8_t* src = a.x + static_cast<uint64_t>(t) * a.x_stride;
    // the first batch of payload vectors does not depend on the routing: fetch it now
    Vec16 v[U];
    if (!quant) {
      #pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t p = team.lane + u * TEAM;
        const uint32_t lv = ll_logical(p);
        if (p < nphys && !ll_is_flag(p) && lv >= hdr_vecs && lv < hdr_vecs + nvec) {
          v[u] = ld_input_v4(src + 16ull * (lv - hdr_vecs));
        }
      }
    }
    // header and scales of the record, as they will appear on the wire
    if (fused_route && team.lane < 32) {
      // the routing is made here: top-k on logit + bias, softmax over the chosen logits
      uint32_t e;
      float w;
      route(t, &e, &w);
      if (team.lane < K) {
        side.hdr[2 + team.lane] = e;
        side.hdr[2 + K + team.lane] = __float_as_uint(w);
        const_cast<uint32_t*>(a.indices)[t * a.indices_stride + team.lane] = e;
        const_cast<float*>(a.weights)[t * a.weights_stride + team.lane] = w;
        atom_relaxed_gpu_add(&ws.route_hist[par * cfg.num_experts + e], 1u);
      }
    }
    for (uint32_t wi = team.lane; wi < hdr_vecs * 4; wi += TEAM) {
      uint32_t word = 0;
      if (wi == 0) word = tag;
      else if (wi == 1) word = static_cast<uint32_t>(t);
      else if (wi < 2u + 2 * K) {
        if (fused_route) continue;
        word = wi < 2u + K ? a.indices[t * a.indices_stride + (wi - 2)]
                           : __float_as_uint(a.weights[t * a.weights_stride + (wi - 2 - K)]);
      }
      side.hdr[wi] = word;
    }
    if (quant) {
      const uint32_t warp_lane = threadIdx.x & 31u;
      const uint32_t lane_base = team.lane - warp_lane;
      #pragma unroll 1
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
          *reinterpret_cast<Vec16*>(side.payload + 16ull * i) = q;
          if ((i & 7u) == 0) *reinterpret_cast<float*>(side.scales + 4 * (i >> 3)) = scale;
        }
      }
      for (uint32_t j = hs + team.lane; j < scale_vecs * 4; j += TEAM) {
        *reinterpret_cast<float*>(side.scales + 4 * j) = 0.f;
      }
    } else {
      const float* xs = reinterpret_cast<const float*>(a.x_scale);
      for (uint32_t j = team.lane; j < scale_vecs * 4; j += TEAM) {
        float val = 0.f;
        if (xs != nullptr && j < static_cast<uint32_t>(hs)) {
          val = xs[t * a.x_scale_stride_token + j * a.x_scale_stride_elem];
        }
        *reinterpret_cast<float*>(side.scales + 4 * j) = val;
      }
    }
    team.sync();
    // one slot per destination rank that owns at least one of the token's experts
    if (team.lane < 32) {
      const int d = team.lane;
      bool hit = false;
      if (d < world && d % cfg.dp_size == my_tp) {
        for (int k = 0; k < K; ++k) {
          const uint32_t e = side.hdr[2 + k];
          hit |= e < static_cast<uint32_t>(cfg.num_experts) && e / L == static_cast<uint32_t>(d);
        }
      }
      uint8_t* rec = nullptr;
      if (hit) {
        if (fused_route) atom_relaxed_gpu_add(&ws.route_nrec[par * kMaxRanks + d], 1u);
        const uint32_t slot = atom_relaxed_gpu_add(&ws.send_cursor[par * kMaxRanks + d], 1u);
        if (slot < static_cast<uint32_t>(cfg.max_num_tokens)) {
          rec = st.recv[d] + cfg.off_drecv + my_group * cfg.drecv_group_stride +
                static_cast<uint64_t>(slot) * cfg.d_stride;
        } else {
          report(ws, kStatusRecordOverflow, kPhaseDispatchSend, d, slot);
        }
      }
      const uint32_t mask = __ballot_sync(0xffffffffu, rec != nullptr);
      if (rec != nullptr) s_dst[team.in_block][__popc(mask & ((1u << d) - 1u))] = rec;
      if (d == 0) s_ndst[team.in_block] = __popc(mask);
    }
    team.sync();
    if (t == 0) trace_mark(cfg, ws, kTraceSendSlots);
    const uint32_t ndst = s_ndst[team.in_block];
    #pragma unroll 1
    for (uint32_t p0 = team.lane; p0 < nphys; p0 += TEAM * U) {
      #pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t p = p0 + u * TEAM;
        if (p >= nphys) continue;
        const uint32_t lv = ll_logical(p);
        if (ll_is_flag(p)) {
          v[u] = flag;
        } else if (lv < hdr_vecs) {
          v[u] = *reinterpret_cast<const Vec16*>(side.hdr + 4 * lv);
        } else if (lv < hdr_vecs + nvec) {
          if (quant) v[u] = *reinterpret_cast<const Vec16*>(side.payload + 16ull * (lv - hdr_vecs));
          else if (p0 != static_cast<uint32_t>(team.lane)) v[u] = ld_input_v4(src + 16ull * (lv - hdr_vecs));
        } else if (lv < hdr_vecs + nvec + scale_vecs) {
          v[u] = *reinterpret_cast<const Vec16*>(side.scales + 16ull * (lv - hdr_vecs - nvec));
        } else {
          v[u] = Vec16{0, 0, 0, 0};
        }
      }
      #pragma unroll 1
      for (uint32_t d = 0; d < ndst; ++d) {
        uint8_t* rec = s_dst[team.in_block][d];
        #pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t p = p0 + u * TEAM;
          if (p < nphys) st_stream_v4(rec + 16ull * p, v[u]);
        }
      }
    }
    if (t == 0) trace_mark(cfg, ws, kTraceSendStored);
    team.sync();  // the side area and the destination list are rewritten by the next token
  }
}

// ---------------------------------------------------------------------------
// dispatch, receiver side: one team per record; every line is taken when its tag is there
// ---------------------------------------------------------------------------

struct RecvLayout {
  const uint32_t* base;        // [G][L] first row of (group, expert), shared memory
  const uint32_t* rec_prefix;  // [kMaxRanks + 1] records before group g
  uint32_t row_cap;
};

__device__ void dispatch_recv_records_ll(const A2AConfig& cfg, const A2ARankState& st,
                                         const DispatchRecvArgs& a, const RecvLayout& lay,
                                         uint32_t tag, uint32_t par, const int TEAM,
                                         uint32_t (*s_rows)[kMaxTopK], uint32_t (*s_unused)[kMaxTopK],
                                         uint32_t* s_nrows, uint8_t* side_base) {
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  const int G = cfg.num_groups;
  const int K = cfg.topk;
  const int L = cfg.experts_per_rank;
  const int rank = st.rank;
  const uint32_t hdr_vecs = cfg.d_header_bytes / 16;
  const uint32_t nvec = cfg.d_payload_bytes / 16;
  const int hs = cfg.hidden_dim_scale;
  const uint32_t scale_vecs = cfg.d_scale_bytes / 16;
  const uint32_t nphys = cfg.d_stride / 16;
  const uint32_t total_recs = lay.rec_prefix[G];
  const uint8_t* drecv = st.recv[rank] + cfg.off_drecv;
  const uint32_t hdr_phys = min(nphys, 32u);  // the header fits the lines one warp covers
  constexpr int U = kLLUnrollDispatch;
  const LLSide side = ll_side(cfg, side_base, team.in_block, false);
  float* os = reinterpret_cast<float*>(a.out_x_scale);

  #pragma unroll 1
  for (uint32_t r = team.id; r < total_recs; r += team.count) {
    int g = 0;
    #pragma unroll
    for (int j = 1; j < kMaxRanks; ++j) {
      if (j < G && r >= lay.rec_prefix[j]) g = j;
    }
    const uint32_t s = r - lay.rec_prefix[g];
    const uint8_t* rec = drecv + g * cfg.drecv_group_stride + static_cast<uint64_t>(s) * cfg.d_stride;
    // Every warp fetches its share of the record's first batch at once (header lines included):
    // a line that is not there yet is simply read again. The header only decides where the
    // payload goes, so nothing waits for it before the payload is in registers.
    const uint32_t warp_first = team.lane & ~31u;  // a warp's 32 vectors are four whole lines
    const uint32_t lane32 = team.lane & 31u;
    Vec16 v[U];
    bool failed = false;
    {
      bool go = true;
      if (team.lane < 32) {
        go = *reinterpret_cast<const volatile uint32_t*>(ws.status) == 0;
        go = __all_sync(0xffffffffu, go);
      }
      if (go && warp_first < nphys) {
        const uint32_t p0 = warp_first + lane32;
        const bool ok = ll_load_lines<U>(
            v, tag, [&](int u) { return rec + 16ull * (p0 + u * TEAM); },
            [&](int u) { return p0 + u * TEAM < nphys; }, cfg.wait_limit_ns, ws.status);
        if (!ok && lane32 == 0) report(ws, kStatusWaitTimeout, kPhaseDispatchRecv, g, r);
        failed = !ok;
      } else {
        failed = !go;
      }
    }
    if (team.lane < 32) {
      const uint32_t p = team.lane;
      bool ok = !failed;
      if (ok && p < hdr_phys && !ll_is_flag(p) && ll_logical(p) < hdr_vecs) {
        *reinterpret_cast<Vec16*>(side.hdr + 4 * ll_logical(p)) = v[0];
      }
      __syncwarp();
      const int k = team.lane;
      uint32_t row = kNoSlot;
      const uint32_t t = ok ? side.hdr[1] : 0u;
      if (ok && t >= static_cast<uint32_t>(cfg.max_num_tokens)) {
        if (k == 0) report(ws, kStatusBadRecord, kPhaseDispatchRecv, g, t);
        ok = false;
      }
      if (ok && k < K) {
        const uint32_t e = side.hdr[2 + k];
        if (e < static_cast<uint32_t>(cfg.num_experts) && e / L == static_cast<uint32_t>(rank)) {
          const int le = e - rank * L;
          row = lay.base[g * L + le] +
                atom_relaxed_gpu_add(&ws.place_cursor[par * (G * L) + g * L + le], 1u);
          if (row < lay.row_cap) {
            ws.row_src[row] = g;
            ws.row_tk[row] = t * K + k;
          } else {
            row = kNoSlot;
          }
        }
        if (cfg.combine_mode == kCombinePreReduce) {
          ws.rec_rows[static_cast<uint64_t>(r) * K + k] = row;
          ws.rec_weights[static_cast<uint64_t>(r) * K + k] = __uint_as_float(side.hdr[2 + K + k]);
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
      #pragma unroll 1
      for (uint32_t w0 = warp_first; w0 < nphys && !failed; w0 += TEAM * U) {
        const uint32_t p0 = w0 + lane32;
        if (w0 != warp_first) {
          const bool ok = ll_load_lines<U>(
              v, tag, [&](int u) { return rec + 16ull * (p0 + u * TEAM); },
              [&](int u) { return p0 + u * TEAM < nphys; }, cfg.wait_limit_ns, ws.status);
          if (!ok) {
            failed = true;
            if (lane32 == 0) report(ws, kStatusWaitTimeout, kPhaseDispatchRecv, g, r);
            break;
          }
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t p = p0 + u * TEAM;
          if (p >= nphys || ll_is_flag(p)) continue;
          const uint32_t lv = ll_logical(p);
          if (lv >= hdr_vecs + nvec) {
            if (lv < hdr_vecs + nvec + scale_vecs) {
              *reinterpret_cast<Vec16*>(side.scales + 16ull * (lv - hdr_vecs - nvec)) = v[u];
            }
          } else if (lv >= hdr_vecs) {
            const uint64_t off = 16ull * (lv - hdr_vecs);
            #pragma unroll 1
            for (uint32_t j = 0; j < nrows; ++j) {
              st_stream_v4(a.out_x + static_cast<uint64_t>(s_rows[team.in_block][j]) * a.out_x_stride + off, v[u]);
            }
          }
        }
      }
      if (hs > 0 && os != nullptr) {
        team.sync();  // the scale vectors of the record are in shared memory now
        const float* sc = reinterpret_cast<const float*>(side.scales);
        #pragma unroll 1
        for (uint32_t i = team.lane; i < nrows * static_cast<uint32_t>(hs); i += TEAM) {
          const uint32_t q = i / hs, j = i - q * hs;
          os[static_cast<int64_t>(s_rows[team.in_block][q]) * a.out_x_scale_stride_token +
             static_cast<int64_t>(j) * a.out_x_scale_stride_elem] = sc[j];
        }
      }
    }
    team.sync();
  }
}

// ---------------------------------------------------------------------------
// combine, sender side
// ---------------------------------------------------------------------------

template <typename Y>
__device__ void combine_send_rows_ll(const A2AConfig& cfg, const A2ARankState& st,
                                     const CombineSendArgs& a, uint32_t tag, uint32_t rows,
                                     uint32_t recs, const int TEAM, uint32_t (*s_rows)[kMaxTopK],
                                     uint32_t (*s_wbits)[kMaxTopK], uint32_t* s_n) {
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  const int K = cfg.topk;
  const uint32_t nvec = static_cast<uint32_t>(cfg.hidden_dim) * cfg.out_elemsize / 16;
  const uint32_t nphys = cfg.c_stride / 16;
  constexpr int U = kLLUnrollCombine;
  const Vec16 flag = {tag, tag, tag, tag};

  if (cfg.combine_mode == kCombinePerRoute) {
    #pragma unroll 1
    for (uint32_t row = team.id; row < rows; row += team.count) {
      const uint8_t* src = a.expert_y + static_cast<uint64_t>(row) * a.expert_y_stride;
      // the row's bytes do not depend on where it goes: fetch the first batch with its destination
      Vec16 v[U];
      auto fetch = [&](uint32_t p0) {
        #pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t p = p0 + u * TEAM;
          v[u] = flag;
          if (p < nphys && !ll_is_flag(p)) {
            const uint32_t lv = ll_logical(p);
            v[u] = lv < nvec ? ld_input_v4(src + 16ull * lv) : Vec16{0, 0, 0, 0};
          }
        }
      };
      fetch(team.lane);
      const uint32_t g = ws.row_src[row];
      const uint32_t tk = ws.row_tk[row];
      if (g == kNoSlot) continue;  // padding row; uniform across the team
      #pragma unroll 1
      for (uint32_t p0 = team.lane; p0 < nphys; p0 += TEAM * U) {
        if (p0 != static_cast<uint32_t>(team.lane)) fetch(p0);
        #pragma unroll 1
        for (int m = 0; m < cfg.dp_size; ++m) {
          uint8_t* dst = st.recv[g * cfg.dp_size + m] + cfg.off_crecv + static_cast<uint64_t>(tk) * cfg.c_stride;
          #pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t p = p0 + u * TEAM;
            if (p < nphys) st_stream_v4(dst + 16ull * p, v[u]);
          }
        }
      }
      if (row == 0) trace_mark(cfg, ws, kTraceCSendStored);
    }
  } else {
    constexpr int N = VecElems<Y>::N;
    constexpr int UP = 4;  // accumulators per lane: UP x 8 floats
    #pragma unroll 1
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
      const uint64_t slot = static_cast<uint64_t>(t) * cfg.world + st.rank;
      #pragma unroll 1
      for (uint32_t p0 = team.lane; p0 < nphys; p0 += TEAM * UP) {
        float acc[UP][8];
        #pragma unroll
        for (int u = 0; u < UP; ++u) {
          #pragma unroll
          for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
        }
        #pragma unroll 1
        for (uint32_t j = 0; j < n; ++j) {
          const uint8_t* row = a.expert_y + static_cast<uint64_t>(s_rows[team.in_block][j]) * a.expert_y_stride;
          const float w = __uint_as_float(s_wbits[team.in_block][j]);
          Vec16 x[UP];
          #pragma unroll
          for (int u = 0; u < UP; ++u) {
            const uint32_t p = p0 + u * TEAM;
            x[u] = Vec16{0, 0, 0, 0};
            if (p < nphys && !ll_is_flag(p) && ll_logical(p) < nvec) x[u] = ld_input_v4(row + 16ull * ll_logical(p));
          }
          #pragma unroll
          for (int u = 0; u < UP; ++u) {
            float f[8];
            VecElems<Y>::unpack(x[u], f);
            #pragma unroll
            for (int q = 0; q < N; ++q) acc[u][q] = fmaf(w, f[q], acc[u][q]);
          }
        }
        #pragma unroll
        for (int u = 0; u < UP; ++u) {
          const uint32_t p = p0 + u * TEAM;
          if (p < nphys) {
            Vec16 out = flag;
            if (!ll_is_flag(p)) {
              uint32_t wds[4];
              VecElems<Y>::pack(acc[u], wds);
              out = Vec16{wds[0], wds[1], wds[2], wds[3]};
            }
            #pragma unroll 1
            for (int m = 0; m < cfg.dp_size; ++m) {
              st_stream_v4(st.recv[g * cfg.dp_size + m] + cfg.off_crecv + slot * cfg.c_stride + 16ull * p, out);
            }
          }
        }
      }
      team.sync();
    }
  }
}

// ---------------------------------------------------------------------------
// combine, receiver side: out[t] = sum_j w_j * row_j, line by line as the lines land
// ---------------------------------------------------------------------------

template <typename Y, typename O>
__device__ void combine_recv_tokens_ll(const A2AConfig& cfg, const A2ARankState& st,
                                       const CombineRecvArgs& a, int T, uint32_t tag, const int TEAM,
                                       uint32_t (*s_slot)[kMaxTopK], uint32_t (*s_wbits)[kMaxTopK],
                                       uint32_t* s_n) {
  const A2ALocal& ws = st.local;
  const Team team(TEAM);
  constexpr int N = VecElems<Y>::N;
  const uint32_t nvec = static_cast<uint32_t>(cfg.hidden_dim) * cfg.out_elemsize / 16;
  const uint32_t nphys = cfg.c_stride / 16;
  const uint8_t* crecv = st.recv[st.rank] + cfg.off_crecv;
  #pragma unroll 1
  for (int t = team.id; t < T; t += team.count) {
    if (team.lane < 32) {
      combine_sources(cfg, a, t, s_slot[team.in_block], s_wbits[team.in_block], &s_n[team.in_block]);
      __syncwarp();
      // stop soon after a failure anywhere on this rank; decided by one lane so that the whole
      // team leaves together
      if (team.lane == 0 && *reinterpret_cast<const volatile uint32_t*>(ws.status) != 0) {
        s_n[team.in_block] = kTeamAbort;
      }
    }
    team.sync();
    const uint32_t n = s_n[team.in_block];
    if (n == kTeamAbort) break;
    uint8_t* out_row = a.out_tokens + static_cast<uint64_t>(t) * a.out_tokens_stride * sizeof(O);
    const uint32_t warp_first = team.lane & ~31u;
    bool failed = false;
    #pragma unroll 1
    for (uint32_t w0 = warp_first; w0 < nphys && !failed; w0 += TEAM) {
      const uint32_t p = w0 + (team.lane & 31u);
      const bool data = p < nphys && !ll_is_flag(p) && ll_logical(p) < nvec;
      const uint64_t elem = static_cast<uint64_t>(ll_logical(p)) * N;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (a.accumulate && data) load_elems<O, N>(out_row, elem, acc);
      #pragma unroll 1
      for (uint32_t j0 = 0; j0 < n; j0 += 8) {
        Vec16 v[8];
        const bool ok = ll_load_lines<8>(
            v, tag,
            [&](int u) { return crecv + static_cast<uint64_t>(s_slot[team.in_block][j0 + u]) * cfg.c_stride + 16ull * p; },
            [&](int u) { return j0 + u < n && p < nphys; }, cfg.wait_limit_ns, ws.status);
        if (!ok) {
          failed = true;
          if ((team.lane & 31u) == 0) report(ws, kStatusWaitTimeout, kPhaseCombineRecv, t, n);
          break;
        }
        #pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (j0 + u < n) {
            const float w = __uint_as_float(s_wbits[team.in_block][j0 + u]);
            float f[8];
            VecElems<Y>::unpack(v[u], f);
            #pragma unroll
            for (int q = 0; q < N; ++q) acc[q] = fmaf(w, f[q], acc[q]);
          }
        }
      }
      if (!failed && data) store_elems<O, N>(out_row, elem, acc);
    }
    if (t == 0) trace_mark(cfg, ws, kTraceCRecvFirstToken);
    team.sync();
  }
}

}  // namespace
}  // namespace pplx
