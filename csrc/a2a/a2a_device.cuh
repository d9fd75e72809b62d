// Device-side helpers shared by the all-to-all kernels: teams, status reporting, bounded
// waits, the end-of-phase bookkeeping, the timeline, 1x128 e4m3 quantisation of a token and
// typed 8-element accessors for the combine arithmetic.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "a2a_types.h"
#include "ptx.cuh"

namespace pplx {
namespace {

constexpr int kMaxTeams = kA2AThreads / 32;
// 16-byte vectors each thread keeps in flight in the copy loops: 512 threads x 8 x 16 B
// = 64 KiB per SM, about what it takes to cover HBM / NVLink latency at full rate.
constexpr int kCopyUnroll = 8;
// Arrival signals (release stores / reductions) a team holds back and publishes together:
// one per lane of its first warp.
constexpr int kMaxPending = 32;

// A team is a power-of-two group of 32..512 consecutive threads of a block that works on
// one token / record / row at a time. Its size is a launch parameter, chosen per phase.
struct Team {
  int size;
  int id;         // global team index inside this virtual rank
  int count;      // teams inside this virtual rank
  int in_block;   // team index inside the block
  int lane;       // thread index inside the team
  __device__ __forceinline__ explicit Team(int team_size) : size(team_size) {
    in_block = threadIdx.x / size;
    lane = threadIdx.x % size;
    // consecutive work items land on different SMs
    id = in_block * gridDim.x + blockIdx.x;
    count = gridDim.x * (kA2AThreads / size);
  }
  __device__ __forceinline__ void sync() const {
    if (size == 32) {
      __syncwarp();
    } else {
      bar_sync(1 + in_block, size);
    }
  }
};

__device__ __forceinline__ void report(const A2ALocal& ws, uint32_t code, uint32_t phase,
                                       uint32_t who, uint32_t detail) {
  if (atomicCAS(&ws.status[0], 0u, code) == 0u) {
    ws.status[1] = phase;
    ws.status[2] = who;
    ws.status[3] = detail;
    *reinterpret_cast<volatile uint32_t*>(ws.host_flag) = code;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* sync_base, int row, int src) {
  // row: see A2AFlagRow; src: the rank that writes the word
  return reinterpret_cast<uint32_t*>(sync_base) + (row * kMaxRanks + src) * kFlagStrideWords;
}

// Bounded wait until a cumulative arrival counter reaches `expected`.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t expected,
                                          uint64_t limit_ns, uint64_t* waited_ns) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - expected) >= 0) {
    *waited_ns = 0;
    return true;
  }
  const uint64_t start = globaltimer_ns();
  for (;;) {
    #pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (static_cast<int32_t>(ld_acquire_sys(flag) - expected) >= 0) {
        *waited_ns = globaltimer_ns() - start;
        return true;
      }
    }
    if (globaltimer_ns() - start > limit_ns) {
      *waited_ns = limit_ns;
      return false;
    }
  }
}

// Marks this block as finished with a *recv* phase (which = 0 dispatch, 1 combine). The
// last block of the launch advances the epoch and clears the placement cursors that the
// dispatch after next will use. Every block read the epoch before it got here, so the
// increment cannot be observed by a block of the same launch.
__device__ __forceinline__ void finish_recv(const A2AConfig& cfg, const A2ALocal& ws, int which,
                                            uint32_t epoch, int trace_slot, bool external) {
  __syncthreads();
  __shared__ uint32_t s_last;
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t old = atom_acq_rel_gpu_add(&ws.done[which], 1u);
    s_last = (old == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    if (which == 0) {
      const int n = cfg.num_groups * cfg.experts_per_rank;
      const uint32_t next_par = (epoch + 1) & 1u;
      for (int i = threadIdx.x; i < n; i += blockDim.x) ws.place_cursor[next_par * n + i] = 0;
    }
    if (threadIdx.x == 0) {
      ws.done[which] = 0;
      ws.epochs[which] = epoch + 1;
      if (external) ws.epochs[2] = ws.epochs[2] + 1;
      if (cfg.trace) ws.trace[trace_slot] = globaltimer_ns();
    }
  }
}

__device__ __forceinline__ uint32_t read_epoch(const A2ALocal& ws, int which) {
  return *reinterpret_cast<volatile const uint32_t*>(&ws.epochs[which]);
}

__device__ __forceinline__ void trace_mark(const A2AConfig& cfg, const A2ALocal& ws, int slot) {
  if (cfg.trace && blockIdx.x == 0 && threadIdx.x == 0) ws.trace[slot] = globaltimer_ns();
}

// Latest time at which any block passed this point.
__device__ __forceinline__ void trace_max(const A2AConfig& cfg, const A2ALocal& ws, int slot) {
  if (cfg.trace && threadIdx.x == 0) atomicMax(&ws.trace[slot], globaltimer_ns());
}


// Quantises 16 consecutive bf16 values (two 16-byte vectors) held by one lane to e4m3;
// eight neighbouring lanes share one 1x128 block and therefore one scale. With `pow2` the scale is
// rounded up to a power of two (what the block-scaled MMA of the expert GEMM can apply itself).
__device__ __forceinline__ Vec16 quantize16(const Vec16& a, const Vec16& b, float* scale_out, bool pow2) {
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float2 f[8];
  float amax = 0.f;
  #pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[i] = __bfloat1622float2(pa[i]);
    f[4 + i] = __bfloat1622float2(pb[i]);
  }
  #pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fmaxf(fabsf(f[i].x), fabsf(f[i].y)));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  float scale = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
  if (pow2) scale = __uint_as_float((__float_as_uint(scale) + 0x007fffffu) & 0x7f800000u);
  const float inv = 1.0f / scale;
  *scale_out = scale;
  Vec16 out;
  uint32_t* o = reinterpret_cast<uint32_t*>(&out);
  #pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 lo = make_float2(f[2 * i].x * inv, f[2 * i].y * inv);
    const float2 hi = make_float2(f[2 * i + 1].x * inv, f[2 * i + 1].y * inv);
    const uint32_t l = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
    const uint32_t h = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
    o[i] = l | (h << 16);
  }
  return out;
}


// Compacts the entries of the team's first warp for which `valid` holds into
// out_a/out_b (shared memory) and returns their number in *out_n. Must be called by
// all 32 lanes of that warp.
__device__ __forceinline__ void compact_warp(bool valid, uint32_t va, uint32_t vb, uint32_t* out_a,
                                             uint32_t* out_b, uint32_t* out_n) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t mask = __ballot_sync(0xffffffffu, valid);
  if (valid) {
    const uint32_t pos = __popc(mask & ((1u << lane) - 1u));
    out_a[pos] = va;
    out_b[pos] = vb;
  }
  if (lane == 0) *out_n = __popc(mask);
}

// Bounded wait until the word at `p` equals `want` (exact = true) or has reached it as a
// counter (exact = false). Gives up when the time limit runs out or when another team of this
// rank has already reported a failure.
__device__ __forceinline__ bool wait_word(const uint32_t* p, uint32_t want, bool exact,
                                          uint64_t limit_ns, const uint32_t* status) {
  auto ok = [&](uint32_t v) { return exact ? v == want : static_cast<int32_t>(v - want) >= 0; };
  if (ok(ld_acquire_sys(p))) return true;
  const uint64_t start = globaltimer_ns();
  for (;;) {
    #pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (ok(ld_acquire_sys(p))) return true;
    }
    if (*reinterpret_cast<const volatile uint32_t*>(status) != 0) return false;
    if (globaltimer_ns() - start > limit_ns) return false;
  }
}

constexpr uint32_t kTeamAbort = 0xfffffffeu;

template <typename T>
struct Elem8;  // 8 consecutive elements as fp32

template <>
struct Elem8<__nv_bfloat16> {
  static constexpr int kBytes = 16;
  __device__ static __forceinline__ void load(const uint8_t* p, float (&f)[8], bool stream) {
    const Vec16 v = stream ? ld_stream_v4(p) : ld_input_v4(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  __device__ static __forceinline__ void store(uint8_t* p, const float (&f)[8]) {
    Vec16 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    st_stream_v4(p, v);
  }
};

template <>
struct Elem8<__half> {
  static constexpr int kBytes = 16;
  __device__ static __forceinline__ void load(const uint8_t* p, float (&f)[8], bool stream) {
    const Vec16 v = stream ? ld_stream_v4(p) : ld_input_v4(p);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __half22float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  __device__ static __forceinline__ void store(uint8_t* p, const float (&f)[8]) {
    Vec16 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
    #pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    st_stream_v4(p, v);
  }
};

template <>
struct Elem8<float> {
  static constexpr int kBytes = 32;
  __device__ static __forceinline__ void load(const uint8_t* p, float (&f)[8], bool stream) {
    const Vec16 a = stream ? ld_stream_v4(p) : ld_input_v4(p);
    const Vec16 b = stream ? ld_stream_v4(p + 16) : ld_input_v4(p + 16);
    f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y);
    f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
    f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y);
    f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
  }
  __device__ static __forceinline__ void store(uint8_t* p, const float (&f)[8]) {
    Vec16 a, b;
    a.x = __float_as_uint(f[0]); a.y = __float_as_uint(f[1]);
    a.z = __float_as_uint(f[2]); a.w = __float_as_uint(f[3]);
    b.x = __float_as_uint(f[4]); b.y = __float_as_uint(f[5]);
    b.z = __float_as_uint(f[6]); b.w = __float_as_uint(f[7]);
    st_stream_v4(p, a);
    st_stream_v4(p + 16, b);
  }
};

// acc += sum_j w[j] * rows[j][granule], eight independent 16/32-byte loads in flight.
template <typename Y>
__device__ __forceinline__ void weighted_gather8(float (&acc)[8], const uint8_t* base,
                                                 uint64_t row_stride, const uint32_t* rows,
                                                 const uint32_t* weights_bits, uint32_t n,
                                                 uint64_t byte_off, bool stream) {
  for (uint32_t j0 = 0; j0 < n; j0 += 8) {
    float f[8][8];
    #pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (j0 + u < n) {
        Elem8<Y>::load(base + static_cast<uint64_t>(rows[j0 + u]) * row_stride + byte_off, f[u],
                       stream);
      }
    }
    #pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (j0 + u < n) {
        const float w = __uint_as_float(weights_bits[j0 + u]);
        #pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = fmaf(w, f[u][q], acc[q]);
      }
    }
  }
}

__device__ __forceinline__ uint32_t* tok_arrive_ptr(const A2AConfig& cfg, uint8_t* sync_base,
                                                    uint32_t t) {
  return reinterpret_cast<uint32_t*>(sync_base + cfg.off_tok_arrive) + t;
}


// ---- ranks outside the NVLink domain (served by the host proxy) ----

__device__ __forceinline__ bool has_remote(const A2AConfig& cfg) {
  return cfg.node_mask != ((cfg.world >= 32) ? 0xffffffffu : ((1u << cfg.world) - 1u));
}

__device__ __forceinline__ bool in_node(const A2AConfig& cfg, uint32_t rank) {
  return ((cfg.node_mask >> rank) & 1u) != 0;
}

// End of a send phase (which = 0 dispatch, 1 combine): the last block to get here tells the host
// proxy, after everything this rank staged has been made visible to the host and to copy
// engines. Called by all threads of every block.
__device__ __forceinline__ void proxy_phase_done(const A2AConfig& cfg, const A2ALocal& ws, int which,
                                                 uint32_t tag) {
  if (!has_remote(cfg)) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t old = atom_acq_rel_gpu_add(&ws.send_done[which], 1u);
    if (old == gridDim.x - 1) {
      ws.send_done[which] = 0;
      volatile uint32_t* words = ws.proxy;
      if (which == 1) {
        for (int g = 0; g < cfg.num_groups; ++g) {
          words[kProxyRows + g] = *reinterpret_cast<volatile uint32_t*>(&ws.stage_cursor[g]);
        }
      }
      __threadfence_system();
      words[which == 0 ? kProxyDispatchSent : kProxyCombineSent] = tag;
    }
  }
}

// How many of token t's combine sources live on ranks inside the NVLink domain (the others are
// announced per rank by the proxy, not per token). First warp of a team, all 32 lanes.
__device__ __forceinline__ uint32_t combine_local_sources(const A2AConfig& cfg, const CombineRecvArgs& a,
                                                          int t) {
  const int K = cfg.topk;
  const int L = cfg.experts_per_rank;
  const int k = threadIdx.x & 31;
  bool counts = false;
  if (k < K) {
    const uint32_t e = a.indices[t * a.indices_stride + k];
    if (e < static_cast<uint32_t>(cfg.num_experts)) {
      const uint32_t d = e / L;
      counts = in_node(cfg, d);
      if (cfg.combine_mode != kCombinePerRoute) {
        for (int q = 0; q < k; ++q) {
          const uint32_t eq = a.indices[t * a.indices_stride + q];
          counts &= !(eq < static_cast<uint32_t>(cfg.num_experts) && eq / L == d);
        }
      }
    }
  }
  return __popc(__ballot_sync(0xffffffffu, counts));
}

// Source slots (and weights) of token t, compacted into shared memory by the first warp
// of the team. *out_n is also the number of arrivals the token waits for.
__device__ __forceinline__ void combine_sources(const A2AConfig& cfg, const CombineRecvArgs& a,
                                                int t, uint32_t* out_slot, uint32_t* out_wbits,
                                                uint32_t* out_n) {
  const int K = cfg.topk;
  const int L = cfg.experts_per_rank;
  const int k = threadIdx.x & 31;
  bool valid = false;
  uint32_t slot = 0, wb = 0;
  if (k < K) {
    const uint32_t e = a.indices[t * a.indices_stride + k];
    if (e < static_cast<uint32_t>(cfg.num_experts)) {
      if (cfg.combine_mode == kCombinePerRoute) {
        valid = true;
        slot = static_cast<uint32_t>(t) * K + k;
        wb = __float_as_uint(a.weights[t * a.weights_stride + k]);
      } else {
        // one partial per distinct destination rank; weights were applied remotely
        const uint32_t d = e / L;
        bool first = true;
        for (int q = 0; q < k; ++q) {
          const uint32_t eq = a.indices[t * a.indices_stride + q];
          first &= !(eq < static_cast<uint32_t>(cfg.num_experts) && eq / L == d);
        }
        valid = first;
        slot = static_cast<uint32_t>(t) * cfg.world + d;
        wb = __float_as_uint(1.0f);
      }
    }
  }
  compact_warp(valid, slot, wb, out_slot, out_wbits, out_n);
}


}  // namespace
}  // namespace pplx
