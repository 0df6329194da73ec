// Peer-memory collectives over NVLink for sm_100a: pull all-gather, pull reduce-scatter with fp32
// accumulation, and a signal-pad barrier between GPUs.  No NCCL: every rank maps every peer's buffers
// (CUDA IPC, set up by the host side below) and the kernels load straight from peer memory with
// system-scope relaxed loads (never through L1).  The kernels use no shared memory and few registers, so
// their CTAs co-reside on the SMs with the persistent tcgen05 GEMM CTAs instead of taking SMs away.
//
// Every wait on another GPU is bounded: when the time limit runs out the kernel records
// YF_ERR_FLAG_TIMEOUT in the status word and returns.
#include <string.h>

#include "common.cuh"
#include "yafsdp_b200.h"

YF_TU_STATUS()

namespace {

constexpr int MAX_RANKS = 16;
struct PeerPtrs {
  void* p[MAX_RANKS];
};

YF_DEVINL uint4 ld_sys_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
YF_DEVINL void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
YF_DEVINL unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// out[r * shard .. (r+1) * shard) = peer_r's shard, for every r.  Rank k starts with its own shard and
// walks the peers in the order k+1, k+2, ...: at any moment every GPU reads from a different peer.
constexpr int AG_UNROLL = 4;
__global__ void __launch_bounds__(512, 1) allgather_pull_kernel(PeerPtrs in, uint4* __restrict__ out, long long shard_vec, int rank, int world) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int d = 0; d < world; ++d) {
    const int r = (rank + d) % world;
    const uint4* src = reinterpret_cast<const uint4*>(in.p[r]);
    uint4* dst = out + (long long)r * shard_vec;
    long long i = tid;
    for (; i + (AG_UNROLL - 1) * stride < shard_vec; i += AG_UNROLL * stride) {
      uint4 v[AG_UNROLL];
#pragma unroll
      for (int u = 0; u < AG_UNROLL; ++u) v[u] = ld_sys_v4(src + i + u * stride);
#pragma unroll
      for (int u = 0; u < AG_UNROLL; ++u) dst[i + u * stride] = v[u];
    }
    for (; i < shard_vec; i += stride) dst[i] = ld_sys_v4(src + i);
  }
}

// dst[i] (+)= scale * sum_{r = 0..world-1} peer_r[rank * shard + i]; the sum runs in rank order on every
// owner, in fp32, so the result is deterministic.  Wire format fp32 or bf16.  WORLD is a template parameter so
// that the per-thread vectors stay in registers; each thread keeps about eight 16-byte peer loads in flight.
template <bool BF16_WIRE, int WORLD>
__global__ void __launch_bounds__(256) reduce_scatter_pull_kernel(PeerPtrs in, float* __restrict__ dst, long long shard_numel, int rank,
                                                                  float scale, int accumulate, float* __restrict__ sumsq) {
  float ss = 0.f;  // squared norm of what this thread writes (gradient-norm fusion, optional)
  constexpr int EPV = BF16_WIRE ? 8 : 4;  // elements per 16-byte vector on the wire
  constexpr int U = (WORLD >= 8) ? 1 : (8 / WORLD);
  const long long nvec = shard_numel / EPV;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const uint4* src[WORLD];
#pragma unroll
  for (int r = 0; r < WORLD; ++r) src[r] = reinterpret_cast<const uint4*>(in.p[r]) + (long long)rank * nvec;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 v[U][WORLD];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) {
#pragma unroll
        for (int r = 0; r < WORLD; ++r) v[u][r] = ld_sys_v4(src[r] + i);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) break;
      float acc[EPV];
#pragma unroll
      for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
#pragma unroll
      for (int r = 0; r < WORLD; ++r) {
        if (BF16_WIRE) {
          const float2 a = unpack_bf16x2(v[u][r].x), b = unpack_bf16x2(v[u][r].y), c = unpack_bf16x2(v[u][r].z),
                       d = unpack_bf16x2(v[u][r].w);
          acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
          acc[4 % EPV] += c.x; acc[5 % EPV] += c.y; acc[6 % EPV] += d.x; acc[7 % EPV] += d.y;
        } else {
          acc[0] += __uint_as_float(v[u][r].x);
          acc[1] += __uint_as_float(v[u][r].y);
          acc[2] += __uint_as_float(v[u][r].z);
          acc[3] += __uint_as_float(v[u][r].w);
        }
      }
      float4* d4 = reinterpret_cast<float4*>(dst + i * EPV);
#pragma unroll
      for (int h = 0; h < EPV / 4; ++h) {
        float4 o = make_float4(acc[4 * h] * scale, acc[4 * h + 1] * scale, acc[4 * h + 2] * scale, acc[4 * h + 3] * scale);
        if (accumulate) {
          const float4 old = d4[h];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        ss += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
        d4[h] = o;
      }
    }
  }
  if (sumsq != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) atomicAdd(sumsq, ss);
  }
}

template <bool BF16_WIRE>
int launch_rs(PeerPtrs pp, float* dst, long long shard_numel, int rank, int world, float scale, int accumulate, int n_ctas,
              float* sumsq, cudaStream_t st) {
  switch (world) {
#define YF_RS_CASE(W)                                                                                                        \
  case W:                                                                                                                    \
    reduce_scatter_pull_kernel<BF16_WIRE, W><<<n_ctas, 256, 0, st>>>(pp, dst, shard_numel, rank, scale, accumulate, sumsq);  \
    return 0;
    YF_RS_CASE(1) YF_RS_CASE(2) YF_RS_CASE(3) YF_RS_CASE(4) YF_RS_CASE(5) YF_RS_CASE(6) YF_RS_CASE(7) YF_RS_CASE(8)
    YF_RS_CASE(9) YF_RS_CASE(10) YF_RS_CASE(11) YF_RS_CASE(12) YF_RS_CASE(13) YF_RS_CASE(14) YF_RS_CASE(15) YF_RS_CASE(16)
#undef YF_RS_CASE
    default:
      return -1;
  }
}

// ---------------------------------------------------------------- NVSwitch multicast (multimem) collectives
// `mc` is the multicast address of a buffer that every rank of the group has bound at the same offset: a store to it
// lands in every rank's copy, a multimem.ld_reduce from it returns the element-wise sum over all ranks' copies,
// computed inside the switch.  Compared with the pull kernels each GPU then receives 1/world of the gradient
// bytes (the reduced stream only) and sends its parameter shard once instead of once per peer.
YF_DEVINL float4 mc_ld_reduce_f32x4(const void* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
YF_DEVINL uint4 mc_ld_reduce_bf16x8(const void* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
YF_DEVINL void mc_st_v4(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// dst[i] (+)= scale * sum over ranks of their buffer[rank * shard + i], the sum taken by the switch.
constexpr int MC_UNROLL = 4;
template <bool BF16_WIRE>
__global__ void __launch_bounds__(256) reduce_scatter_mc_kernel(const char* __restrict__ mc_in, float* __restrict__ dst, long long shard_numel,
                                                                int rank, float scale, int accumulate, float* __restrict__ sumsq) {
  constexpr int EPV = BF16_WIRE ? 8 : 4;
  const long long nvec = shard_numel / EPV;
  const char* src = mc_in + (long long)rank * shard_numel * (BF16_WIRE ? 2 : 4);
  const long long stride = (long long)gridDim.x * blockDim.x;
  float ss = 0.f;
  auto finish = [&](long long v, float4 o) {
    float4* d4 = reinterpret_cast<float4*>(dst) + v;
    o.x *= scale; o.y *= scale; o.z *= scale; o.w *= scale;
    if (accumulate) {
      const float4 old = *d4;
      o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
    }
    ss += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
    *d4 = o;
  };
  for (long long base = blockIdx.x * (long long)blockDim.x + threadIdx.x; base < nvec; base += MC_UNROLL * stride) {
    if constexpr (BF16_WIRE) {
      uint4 raw[MC_UNROLL];
#pragma unroll
      for (int u = 0; u < MC_UNROLL; ++u)
        if (base + u * stride < nvec) raw[u] = mc_ld_reduce_bf16x8(src + (base + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < MC_UNROLL; ++u) {
        const long long v = base + u * stride;
        if (v >= nvec) continue;
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f[2 * j] = __uint_as_float(w[j] << 16);
          f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
        finish(2 * v, make_float4(f[0], f[1], f[2], f[3]));
        finish(2 * v + 1, make_float4(f[4], f[5], f[6], f[7]));
      }
    } else {
      float4 acc[MC_UNROLL];
#pragma unroll
      for (int u = 0; u < MC_UNROLL; ++u)
        if (base + u * stride < nvec) acc[u] = mc_ld_reduce_f32x4(src + (base + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < MC_UNROLL; ++u)
        if (base + u * stride < nvec) finish(base + u * stride, acc[u]);
    }
  }
  if (sumsq != nullptr) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) atomicAdd(sumsq, ss);
  }
}

// Every rank's copy of out[rank * shard .. (rank + 1) * shard) = this rank's shard: one multicast store per 16 bytes.
__global__ void __launch_bounds__(256) allgather_mc_kernel(const uint4* __restrict__ in, char* __restrict__ mc_out, long long shard_vec, int rank) {
  char* dst = mc_out + (long long)rank * shard_vec * 16;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long base = blockIdx.x * (long long)blockDim.x + threadIdx.x; base < shard_vec; base += MC_UNROLL * stride) {
    uint4 v[MC_UNROLL];
#pragma unroll
    for (int u = 0; u < MC_UNROLL; ++u)
      if (base + u * stride < shard_vec) v[u] = in[base + u * stride];
#pragma unroll
    for (int u = 0; u < MC_UNROLL; ++u)
      if (base + u * stride < shard_vec) mc_st_v4(dst + (base + u * stride) * 16, v[u]);
  }
}

// Push a contiguous range of the flat layer gradient (fp32, `numel` elements starting at flat position `flat_off`) into the
// reduce-scatter slots of the ranks that own it: element f goes to peer_grad[f / shard] + rank * shard + f % shard.  A null
// source pushes zeros.  For the small gradients (norm weights, biases) that no GEMM epilogue produces.
template <bool BF16_WIRE>
__global__ void __launch_bounds__(256) push_flat_kernel(const float4* __restrict__ src, long long nvec, long long flat_off, PeerPtrs peer_grad,
                                                        long long shard_numel, int rank) {
  constexpr int EPV = BF16_WIRE ? 8 : 4;  // elements per 16-byte piece on the wire
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const long long f = flat_off + i * EPV;
    const long long o = f / shard_numel;
    const long long loc = f - o * shard_numel;
#ifdef YF_DEBUG_BOUNDS
    if (o < 0 || o >= MAX_RANKS || peer_grad.p[o] == nullptr || loc + EPV > shard_numel) {  // debug build: record and skip
      yf_raise(YF_ERR_BAD_ARGUMENT, 41);
      continue;
    }
#endif
    if (BF16_WIRE) {
      const float4 a = src != nullptr ? src[2 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 b = src != nullptr ? src[2 * i + 1] : make_float4(0.f, 0.f, 0.f, 0.f);
      const uint4 v = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_grad.p[o]) + (long long)rank * shard_numel + loc) = v;
    } else {
      const float4 v = src != nullptr ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(peer_grad.p[o]) + (long long)rank * shard_numel + loc) = v;
    }
  }
}

// Signal pads.  Layout: unsigned 64-bit words [slot][MAX_RANKS] in every rank's pad; rank k owns word [slot][k] of every
// pad and only ever raises it (atomic max), so sequence numbers are monotonic even when two streams signal the same slot
// and pads are never reset.
YF_DEVINL void red_max_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.max.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// one thread per peer: raise word [slot][rank] of that peer's pad to `seq`
YF_DEVINL void pad_signal(const PeerPtrs& pads, int r, int rank, int slot, unsigned long long seq) {
  __threadfence_system();
  red_max_release_sys_u64(reinterpret_cast<unsigned long long*>(pads.p[r]) + (size_t)slot * MAX_RANKS + rank, seq);
}
// one thread per peer: wait (bounded) until word [slot][r] of this rank's own pad has reached `seq`
YF_DEVINL void pad_wait(const PeerPtrs& pads, int r, int rank, int slot, unsigned long long seq, unsigned long long timeout_ns) {
  const unsigned long long* mine = reinterpret_cast<const unsigned long long*>(pads.p[rank]) + (size_t)slot * MAX_RANKS + r;
  const uint64_t t0 = yf_globaltimer();
  for (uint32_t it = 0;; ++it) {
    if (ld_acquire_sys_u64(mine) >= seq) break;
    if ((it & 63u) == 63u) {
      if (yf_aborted() || yf_globaltimer() - t0 > timeout_ns) {
        yf_raise(YF_ERR_FLAG_TIMEOUT, 300 + slot);
        break;
      }
      __nanosleep(200);
    }
  }
  __threadfence_system();
}
// mode bit 0: signal, bit 1: wait.  Both = a barrier between the GPUs' streams; signal alone tells the peers that this
// rank's stream got here; wait alone blocks this stream until every peer's signal `seq` has arrived.
__global__ void signal_pad_kernel(PeerPtrs pads, int rank, int world, int slot, unsigned long long seq, unsigned long long timeout_ns,
                                  int mode) {
  const int r = threadIdx.x;
  if (r >= world) return;
  if (mode & 1) pad_signal(pads, r, rank, slot, seq);
  if (mode & 2) pad_wait(pads, r, rank, slot, seq, timeout_ns);
}

// Wait until word `index` of a local flag array reaches `value` (bounded); and its setter.
__global__ void flag_wait_kernel(const unsigned long long* flags, long long index, unsigned long long value, unsigned long long timeout_ns) {
  const uint64_t t0 = yf_globaltimer();
  for (uint32_t it = 0;; ++it) {
    if (ld_acquire_sys_u64(flags + index) >= value) break;
    if ((it & 63u) == 63u) {
      if (yf_globaltimer() - t0 > timeout_ns) {
        yf_raise(YF_ERR_FLAG_TIMEOUT, 400);
        break;
      }
      __nanosleep(200);
    }
  }
}
__global__ void flag_set_kernel(unsigned long long* flags, long long index, unsigned long long value) {
  __threadfence_system();
  st_release_sys_u64(flags + index, value);
}

PeerPtrs to_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

}  // namespace

extern "C" int yf_allgather_pull(void* const* peer_in, void* out, long long shard_bytes, int rank, int world, int n_ctas, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || shard_bytes <= 0 || (shard_bytes % 16)) return -1;
  if (reinterpret_cast<uintptr_t>(out) & 15) return -1;
  for (int r = 0; r < world; ++r)
    if (!peer_in[r] || (reinterpret_cast<uintptr_t>(peer_in[r]) & 15)) return -1;
  // one CTA per SM: 512 threads x <= 64 registers leaves room for a persistent GEMM CTA on the same SM
  if (n_ctas <= 0) n_ctas = yf_num_sms();
  allgather_pull_kernel<<<n_ctas, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(to_peers(peer_in, world), reinterpret_cast<uint4*>(out),
                                                                                   shard_bytes / 16, rank, world);
  return -(int)cudaGetLastError();
}

extern "C" int yf_reduce_scatter_pull_sumsq(void* const* peer_in, float* dst, long long shard_numel, int rank, int world, float scale,
                                            int accumulate, int bf16_wire, int n_ctas, float* sumsq, void* stream);

extern "C" int yf_reduce_scatter_pull(void* const* peer_in, float* dst, long long shard_numel, int rank, int world, float scale,
                                      int accumulate, int bf16_wire, int n_ctas, void* stream) {
  return yf_reduce_scatter_pull_sumsq(peer_in, dst, shard_numel, rank, world, scale, accumulate, bf16_wire, n_ctas, nullptr, stream);
}

// Same; when `sumsq` is given the kernel also adds the squared norm of the values it leaves in dst to *sumsq.
extern "C" int yf_reduce_scatter_pull_sumsq(void* const* peer_in, float* dst, long long shard_numel, int rank, int world, float scale,
                                            int accumulate, int bf16_wire, int n_ctas, float* sumsq, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || shard_numel <= 0 || (shard_numel % 8)) return -1;
  if (reinterpret_cast<uintptr_t>(dst) & 15) return -1;
  for (int r = 0; r < world; ++r)
    if (!peer_in[r] || (reinterpret_cast<uintptr_t>(peer_in[r]) & 15)) return -1;
  if (n_ctas <= 0) n_ctas = yf_num_sms();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PeerPtrs pp = to_peers(peer_in, world);
  const int rc = bf16_wire ? launch_rs<true>(pp, dst, shard_numel, rank, world, scale, accumulate, n_ctas, sumsq, st)
                           : launch_rs<false>(pp, dst, shard_numel, rank, world, scale, accumulate, n_ctas, sumsq, st);
  if (rc != 0) return rc;
  return -(int)cudaGetLastError();
}

// Reduce-scatter through the switch: `mc_in` is the multicast address of the (fp32 or bf16) gradient buffer.
extern "C" int yf_reduce_scatter_mc(const void* mc_in, float* dst, long long shard_numel, int rank, int world, float scale, int accumulate,
                                    int bf16_wire, int n_ctas, float* sumsq, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || shard_numel <= 0 || (shard_numel % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(mc_in) & 15) || mc_in == nullptr) return -1;
  if (n_ctas <= 0) n_ctas = 64;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bf16_wire)
    reduce_scatter_mc_kernel<true><<<n_ctas, 256, 0, st>>>(static_cast<const char*>(mc_in), dst, shard_numel, rank, scale, accumulate, sumsq);
  else
    reduce_scatter_mc_kernel<false><<<n_ctas, 256, 0, st>>>(static_cast<const char*>(mc_in), dst, shard_numel, rank, scale, accumulate, sumsq);
  return -(int)cudaGetLastError();
}

// All-gather through the switch: this rank's shard is stored once to the multicast address of the output buffer.
extern "C" int yf_allgather_mc(const void* in, void* mc_out, long long shard_bytes, int rank, int world, int n_ctas, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || shard_bytes <= 0 || (shard_bytes & 15)) return -1;
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(mc_out) & 15) || mc_out == nullptr) return -1;
  if (n_ctas <= 0) n_ctas = 32;
  allgather_mc_kernel<<<n_ctas, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(in), static_cast<char*>(mc_out),
                                                                                 shard_bytes / 16, rank);
  return -(int)cudaGetLastError();
}

extern "C" int yf_push_flat(const float* src, long long numel, long long flat_off, void* const* peer_grad, long long shard_numel, int rank,
                            int world, int wire_bf16, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || numel <= 0) return -1;
  const int epv = wire_bf16 ? 8 : 4;
  if ((numel % epv) || (flat_off % epv) || (shard_numel % epv) || flat_off < 0 || flat_off + numel > shard_numel * world) return -1;
  if (reinterpret_cast<uintptr_t>(src) & 15) return -1;
  for (int r = 0; r < world; ++r)
    if (!peer_grad[r] || (reinterpret_cast<uintptr_t>(peer_grad[r]) & 15)) return -1;
  const long long nvec = numel / epv;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 2 * yf_num_sms()) blocks = 2 * yf_num_sms();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (wire_bf16)
    push_flat_kernel<true><<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const float4*>(src), nvec, flat_off, to_peers(peer_grad, world),
                                                       shard_numel, rank);
  else
    push_flat_kernel<false><<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const float4*>(src), nvec, flat_off, to_peers(peer_grad, world),
                                                        shard_numel, rank);
  return -(int)cudaGetLastError();
}

extern "C" int yf_signal_pad(void* const* pads, int rank, int world, int slot, long long seq, long long timeout_ms, int mode,
                             void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || slot < 0 || seq <= 0 || (mode & 3) == 0) return -1;
  if (int rc = yf_tu_bind_status()) return rc;
  signal_pad_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(to_peers(pads, world), rank, world, slot, (unsigned long long)seq,
                                                                         (unsigned long long)timeout_ms * 1000000ull, mode & 3);
  return -(int)cudaGetLastError();
}

extern "C" int yf_signal_barrier(void* const* pads, int rank, int world, int slot, long long seq, long long timeout_ms, void* stream) {
  return yf_signal_pad(pads, rank, world, slot, seq, timeout_ms, 3, stream);
}

extern "C" int yf_flag_wait(const void* flags, long long index, long long value, long long timeout_ms, void* stream) {
  if (int rc = yf_tu_bind_status()) return rc;
  flag_wait_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const unsigned long long*>(flags), index,
                                                                       (unsigned long long)value, (unsigned long long)timeout_ms * 1000000ull);
  return -(int)cudaGetLastError();
}

extern "C" int yf_flag_set(void* flags, long long index, long long value, void* stream) {
  flag_set_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<unsigned long long*>(flags), index,
                                                                      (unsigned long long)value);
  return -(int)cudaGetLastError();
}

// ---------------------------------------------------------------- peer-mapped memory (CUDA IPC)
// yf_ipc_alloc: cudaMalloc + zero + export handle (64 bytes).  yf_ipc_open: map a peer's handle into this
// process (peer access is enabled lazily by the runtime).  Allocations live until yf_ipc_free / process exit.
extern "C" int yf_ipc_alloc(long long nbytes, void** ptr_out, void* handle_out64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)nbytes);
  if (e != cudaSuccess) return -(int)e;
  e = cudaMemset(p, 0, (size_t)nbytes);
  if (e != cudaSuccess) return -(int)e;
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return -(int)e;
  memcpy(handle_out64, &h, sizeof(h));
  *ptr_out = p;
  return 0;
}
extern "C" int yf_ipc_open(const void* handle64, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return -(int)e;
  *ptr_out = p;
  return 0;
}
extern "C" int yf_ipc_close(void* ptr) { return -(int)cudaIpcCloseMemHandle(ptr); }
extern "C" int yf_ipc_free(void* ptr) { return -(int)cudaFree(ptr); }
