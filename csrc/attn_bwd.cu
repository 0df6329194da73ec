// Causal flash-attention backward for head_dim 128 on sm_100a (MHA and GQA).
//
// One CTA per (128-key tile, KV head, sequence); it walks the query tiles (and, for GQA, the query
// heads of the group) that attend to those keys.  Per step five tcgen05 GEMMs:
//   S  = Q K^T          dP = dO V^T                    (fp32 in TMEM, one query row per TMEM lane)
//   P  = exp(S*scale - lse),  dS = P * (dP - D) * scale   (softmax warps; bf16 into swizzled smem)
//   dV += P^T dO        dK += dS^T Q                   (accumulated in TMEM over the whole walk)
//   dQ_part = dS K      -> staged in shared memory, added to a global fp32 dQ accumulator by TMA reduce-add
// The P / dS tiles are stored once as [query][key] with the 128-byte swizzle and are read both as a
// K-major operand (dQ) and as an MN-major operand (dV, dK): the two canonical layouts coincide.
// D = rowsum(dO * O) comes from a small pre-pass; dQ is converted to bf16 by a post-pass.
#include <stdio.h>

#include "common.cuh"
#include "yafsdp_b200.h"

YF_TU_STATUS()

namespace {

constexpr int HD = 128;
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int ATOM = 16384;
constexpr int TILE = 2 * ATOM;
constexpr int BWD_THREADS = 320;  // producer warp, MMA warp, eight softmax / epilogue warps
constexpr int BWD_SMEM = 1024 + 7 * TILE + 256;  // K, V, Q, dO, P, dS and the dQ staging (two [128 x 32 fp32] blocks)

struct BwdArgs {
  const float* lse;    // [B, Hq, S]
  const float* delta;  // [B, Hq, S]
  float* dq_accum;     // [B*S, Hq*128] fp32, zeroed by the caller
  __nv_bfloat16* dk;   // rows dkv_stride apart, head hk at columns hk*128
  __nv_bfloat16* dv;
  long long dkv_stride;
  int S, B, Hq, Hkv;
  float scale, scale_log2;
  int causal;
};

YF_DEVINL void tma_reduce_add_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_do,
                const __grid_constant__ CUtensorMap tma_dq, BwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;
  uint8_t* sdO = sQ + TILE;
  uint8_t* sP = sdO + TILE;
  uint8_t* sdS = sP + TILE;
  uint8_t* sdQ = sdS + TILE;  // two 16 KB blocks, 128-byte swizzled rows, source of the TMA reduce-adds
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdQ + TILE);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_ready = bars + 4;
  uint64_t* dq_full = bars + 5;
  uint64_t* dq_read = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int jt = blockIdx.x;  // key tile
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int group = args.Hq / args.Hkv;
  const int kv0 = jt * BKV;
  const int nq_tiles = (args.S + BQ - 1) / BQ;
  const int i_start = args.causal ? jt : 0;
  const int per_head = nq_tiles - i_start;
  const int n_it = per_head * group;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
    tma_prefetch_desc(&tma_do);
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_read, 256);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE);
      tma_load_3d(sK, &tma_k, kv_full, hk * HD, kv0, b);
      tma_load_3d(sK + ATOM, &tma_k, kv_full, hk * HD + 64, kv0, b);
      tma_load_3d(sV, &tma_v, kv_full, hk * HD, kv0, b);
      tma_load_3d(sV + ATOM, &tma_v, kv_full, hk * HD + 64, kv0, b);
      for (int it = 0; it < n_it; ++it) {
        const int h = hk * group + it / per_head;
        const int q0 = (i_start + it % per_head) * BQ;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, 200)) break;
        mbar_expect_tx(qdo_full, 2 * TILE);
        tma_load_3d(sQ, &tma_q, qdo_full, h * HD, q0, b);
        tma_load_3d(sQ + ATOM, &tma_q, qdo_full, h * HD + 64, q0, b);
        tma_load_3d(sdO, &tma_do, qdo_full, h * HD, q0, b);
        tma_load_3d(sdO + ATOM, &tma_do, qdo_full, h * HD + 64, q0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = umma_idesc_bf16(128, 128, 0, 0);
      const uint32_t id_mm = umma_idesc_bf16(128, 128, 1, 1);
      const uint32_t id_km = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO), aP = smem_u32(sP),
                     adS = smem_u32(sdS);
      bool alive = mbar_wait(kv_full, 0, 210);
      for (int it = 0; it < n_it && alive; ++it) {
        if (!mbar_wait(qdo_full, it & 1, 211)) { alive = false; break; }
        if (it > 0 && !mbar_wait(dq_read, (it - 1) & 1, 212)) { alive = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // S = Q K^T
          const uint32_t off = (k >> 2) * ATOM + (k & 3) * 32;
          tc_mma_bf16(tS, umma_smem_desc_sw128(aQ + off, 0, 1024), umma_smem_desc_sw128(aK + off, 0, 1024), id_kk, k != 0);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // dP = dO V^T
          const uint32_t off = (k >> 2) * ATOM + (k & 3) * 32;
          tc_mma_bf16(tdP, umma_smem_desc_sw128(adO + off, 0, 1024), umma_smem_desc_sw128(aV + off, 0, 1024), id_kk, k != 0);
        }
        tc_commit(sdp_full);
        if (!mbar_wait(pds_ready, it & 1, 213)) { alive = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dV += P^T dO   (A = P read MN-major, B = dO MN-major; K = query rows)
          tc_mma_bf16(tdV, umma_smem_desc_sw128(aP + k * 2048, ATOM, 1024), umma_smem_desc_sw128(adO + k * 2048, ATOM, 1024),
                      id_mm, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dK += dS^T Q
          tc_mma_bf16(tdK, umma_smem_desc_sw128(adS + k * 2048, ATOM, 1024), umma_smem_desc_sw128(aQ + k * 2048, ATOM, 1024),
                      id_mm, (it | k) != 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // dQ_part = dS K   (A = dS K-major over keys, B = K tile MN-major)
          tc_mma_bf16(tS, umma_smem_desc_sw128(adS + (k >> 2) * ATOM + (k & 3) * 32, 0, 1024),
                      umma_smem_desc_sw128(aK + k * 2048, ATOM, 1024), id_km, k != 0);
        tc_commit(dq_full);
        tc_commit(qdo_empty);
      }
    }
  } else {
    // eight warps: warp w owns TMEM lanes [32*(w%4), +32) (one query row per thread) and, of the four 32-column
    // chunks of every tile, the two of its half ((w-2)/4): two threads share a row and split its columns
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int c_begin = ((warp - 2) >> 2) * 2, c_end = c_begin + 2;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const float sl2 = args.scale_log2;
    bool alive = true;
    for (int it = 0; it < n_it && alive; ++it) {
      const int h = hk * group + it / per_head;
      const int q0 = (i_start + it % per_head) * BQ;
      const int qrow = q0 + row;
      const bool row_ok = qrow < args.S;
      const long long stat_idx = ((long long)b * args.Hq + h) * args.S + qrow;
      const float lse2 = row_ok ? args.lse[stat_idx] * 1.4426950408889634f : 0.f;
      const float delta = row_ok ? args.delta[stat_idx] : 0.f;
      // keys this query row may see: col <= limit
      const int limit = row_ok ? (args.causal ? min(qrow, args.S - 1) : args.S - 1) : -1;
      const bool need_mask = kv0 + BKV - 1 > limit;
      if (!mbar_wait(sdp_full, it & 1, 220)) { alive = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(tS + lane_off + c * 32, rs);
        tmem_ld32(tdP + lane_off + c * 32, rp);
        tmem_ld_wait();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(rs[t]), sl2, -lse2));
          float p1 = fast_exp2(fmaf(__uint_as_float(rs[t + 1]), sl2, -lse2));
          if (need_mask) {  // only the tiles on the diagonal and the last one have masked keys
            if (kv0 + c * 32 + t > limit) p0 = 0.f;
            if (kv0 + c * 32 + t + 1 > limit) p1 = 0.f;
          }
          const float d0 = p0 * (__uint_as_float(rp[t]) - delta) * args.scale;
          const float d1 = p1 * (__uint_as_float(rp[t + 1]) - delta) * args.scale;
          pk[t >> 1] = pack_bf16x2(p0, p1);
          dk[t >> 1] = pack_bf16x2(d0, d1);
        }
        const int tile_off = (c >> 1) * ATOM + row * 128;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int chunk = (((c & 1) * 4 + t) ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(sP + tile_off + chunk) = make_uint4(pk[4 * t], pk[4 * t + 1], pk[4 * t + 2], pk[4 * t + 3]);
          *reinterpret_cast<uint4*>(sdS + tile_off + chunk) = make_uint4(dk[4 * t], dk[4 * t + 1], dk[4 * t + 2], dk[4 * t + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_ready);
      if (!mbar_wait(dq_full, it & 1, 221)) { alive = false; break; }
      tc_fence_after();
      // dQ_part: TMEM -> registers -> swizzled staging block -> one TMA reduce-add per [128 rows x 32 columns] block (full
      // 128-byte lines reach the L2 reduction units; rows past the end of the sequence are clipped by the tensor map).
      // The two column halves of the tile use one staging block each; two passes cover the four 32-column chunks.
      const bool dq_thread = (threadIdx.x == 64 || threadIdx.x == 64 + 128);  // first thread of each half
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        const int c = c_begin + pass;
        uint8_t* blk = sdQ + (c_begin >> 1) * ATOM;  // half 0 -> block 0, half 1 -> block 1
        uint32_t r[32];
        tmem_ld32(tS + lane_off + c * 32, r);
        tmem_ld_wait();
        if (dq_thread) tma_store_wait_read0();  // the reduce that last read this block has finished reading
        named_bar_sync(2 + (c_begin >> 1), 128);
        uint8_t* srow = blk + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        fence_proxy_async_smem();
        named_bar_sync(2 + (c_begin >> 1), 128);
        if (dq_thread) {
          tma_reduce_add_3d(&tma_dq, blk, h * HD + c * 32, q0, b);
          tma_store_commit();
        }
      }
      tc_fence_before();
      mbar_arrive(dq_read);
    }
    if (threadIdx.x == 64 || threadIdx.x == 64 + 128) tma_store_wait0();  // this thread's dQ reduce-adds have completed
    // dK, dV: TMEM lane == key row.  The last dq_full wait covers every MMA issued before it.
    if (alive) {  // every lane issues the (warp-collective) TMEM loads; only the stores are predicated
      const bool key_ok = kv0 + row < args.S;
      const long long off = ((long long)b * args.S + kv0 + row) * args.dkv_stride + hk * HD;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? args.dv : args.dk) + off;
        const uint32_t tsrc = (which == 0 ? tdV : tdK) + lane_off;
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[32];
          tmem_ld32(tsrc + c * 32, r);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              w.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              w.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              w.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              reinterpret_cast<uint4*>(dst + c * 32)[v] = w;
            }
          }
        }
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,s] = sum_d dO * O, and the fp32 dQ accumulator of the same (token, head) cleared on the way (the main kernel
// adds into it): sixteen lanes per (token, head), one 16-byte load of O and of dO and two 16-byte stores of zeros per lane.
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                                         float* __restrict__ delta, float* __restrict__ dq_zero, int B, int S, int Hq,
                                                         long long o_stride, long long do_stride) {
  const long long total = (long long)B * S * Hq;
  const int sub = threadIdx.x & 15;
  const unsigned half_mask = 0xffffu << (threadIdx.x & 16);  // the two halves of a warp may leave the loop at different times
  for (long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 4; w < total;
       w += ((long long)gridDim.x * blockDim.x) >> 4) {
    const int h = (int)(w % Hq);
    const long long t = w / Hq;
    const uint4 a = *reinterpret_cast<const uint4*>(o + t * o_stride + h * HD + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + t * do_stride + h * HD + sub * 8);
    if (dq_zero != nullptr) {
      float4* z = reinterpret_cast<float4*>(dq_zero + (t * Hq + h) * HD + sub * 8);
      z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
    float s = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y + a3.x * g3.x + a3.y * g3.y;
#pragma unroll
    for (int m = 8; m >= 1; m >>= 1) s += __shfl_xor_sync(half_mask, s, m);
    if (sub == 0) {
      const long long bb = t / S, ss = t % S;
      delta[(bb * Hq + h) * S + ss] = s;
    }
  }
}

// dq (bf16, strided rows) = dq_accum (fp32, dense rows of `width`)
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long T, int width,
                                       long long dq_stride) {
  const int vpr = width / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    const float4 a = reinterpret_cast<const float4*>(acc + t * width)[2 * v];
    const float4 c = reinterpret_cast<const float4*>(acc + t * width)[2 * v + 1];
    uint4 w;
    w.x = pack_bf16x2(a.x, a.y);
    w.y = pack_bf16x2(a.z, a.w);
    w.z = pack_bf16x2(c.x, c.y);
    w.w = pack_bf16x2(c.z, c.w);
    *reinterpret_cast<uint4*>(dq + t * dq_stride + v * 8) = w;
  }
}

}  // namespace

// The three launches of one backward pass (delta pre-pass, main kernel, dQ conversion), shared by both entry points.
// Allocates nothing: the tensor maps come by reference from the caller, the scratch by pointer.
static int attn_bwd_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& md,
                           const CUtensorMap& mdq, const void* out,
                           const void* dout, const float* lse, float* delta, float* dq_accum, void* dq, void* dk, void* dv, int B,
                           int S, int Hq, int Hkv, long long o_stride, long long do_stride, long long dq_stride,
                           long long dkv_stride, float scale, int causal, cudaStream_t st) {
  static bool optin[64] = {};  // the shared-memory opt-in is a per-device attribute
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!optin[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e != cudaSuccess) return -(int)e;
    optin[dev] = true;
  }
  if (int rc = yf_tu_bind_status()) return rc;
  const long long T = (long long)B * S;
  {
    // delta pre-pass; it also clears the dQ accumulator, which must start at zero on every call
    const long long groups = T * Hq;
    long long blocks = (groups * 16 + 255) / 256;
    const long long cap = (long long)yf_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    attn_delta_kernel<<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                  reinterpret_cast<const __nv_bfloat16*>(dout), delta, dq_accum, B, S, Hq, o_stride,
                                                  do_stride);
  }
  BwdArgs a;
  a.lse = lse;
  a.delta = delta;
  a.dq_accum = dq_accum;
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  a.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  a.dkv_stride = dkv_stride;
  a.S = S; a.B = B; a.Hq = Hq; a.Hkv = Hkv;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal ? 1 : 0;
  dim3 grid((S + BKV - 1) / BKV, Hkv, B);
  attn_bwd_kernel<<<grid, BWD_THREADS, BWD_SMEM, st>>>(mq, mk, mv, md, mdq, a);
  {
    const long long items = T * (Hq * HD / 8);
    long long blocks = (items + 255) / 256;
    const long long cap = (long long)yf_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    attn_dq_convert_kernel<<<(int)blocks, 256, 0, st>>>(dq_accum, reinterpret_cast<__nv_bfloat16*>(dq), T, Hq * HD, dq_stride);
  }
  return -(int)cudaGetLastError();
}

// Backward of yf_attn_fwd.  q/k/v/out/dout as in the forward (dout rows do_stride apart, out rows
// o_stride apart); lse from the forward.  Scratch supplied by the caller: delta [B,Hq,S] fp32 and
// dq_accum [B*S, Hq*128] fp32 (zeroed here).  Results: dq (rows dq_stride apart), dk/dv (rows
// dkv_stride apart), all bf16; they may be column blocks of one fused d(QKV) buffer.
extern "C" int yf_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                           float* delta, float* dq_accum, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv,
                           long long q_stride, long long kv_stride, long long o_stride, long long do_stride,
                           long long dq_stride, long long dkv_stride, float scale, int causal, void* stream) {
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv)) return -1;
  if ((q_stride % 8) || (kv_stride % 8) || (o_stride % 8) || (do_stride % 8) || (dq_stride % 8) || (dkv_stride % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) |
       reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(dq_accum)) & 15)
    return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const CUtensorMap* mq = yf_tensor_map_3d(q, (uint64_t)Hq * HD, S, B, q_stride, (uint64_t)S * q_stride, 64, BQ, 1, 2, 1);
  const CUtensorMap* mk = yf_tensor_map_3d(k, (uint64_t)Hkv * HD, S, B, kv_stride, (uint64_t)S * kv_stride, 64, BKV, 1, 2, 1);
  const CUtensorMap* mv = yf_tensor_map_3d(v, (uint64_t)Hkv * HD, S, B, kv_stride, (uint64_t)S * kv_stride, 64, BKV, 1, 2, 1);
  const CUtensorMap* md = yf_tensor_map_3d(dout, (uint64_t)Hq * HD, S, B, do_stride, (uint64_t)S * do_stride, 64, BQ, 1, 2, 1);
  const CUtensorMap* mdq = yf_tensor_map_3d(dq_accum, (uint64_t)Hq * HD, S, B, (uint64_t)Hq * HD, (uint64_t)S * Hq * HD, 32, BQ, 1, 4, 1);
  if (!mq || !mk || !mv || !md || !mdq) return -2;
  return attn_bwd_launch(*mq, *mk, *mv, *md, *mdq, out, dout, lse, delta, dq_accum, dq, dk, dv, B, S, Hq, Hkv, o_stride, do_stride, dq_stride,
                         dkv_stride, scale, causal, st);
}

// ------------------------------------------------------------------------------------------------
// yf_attn_bwd_noalloc: the same backward for callers that cannot allocate device memory.
//
// yf_attn_bwd needs two scratch arrays from its caller (delta and the fp32 dQ accumulator).  Some users of
// this library have no way to provide them: a C or C++ host that binds the exported symbols without a
// tensor framework, or a job that hands all of the GPU's memory to its own pool at start-up, where a later
// cudaMalloc fails and a borrowed pool block is not available to a third-party call.  For them the scratch
// lives in the fixed device array below, which every GPU that loads this library holds until the process
// exits (about 16.1 MiB).  Nothing here calls cudaMalloc, cudaFree, a framework allocator or the tensor-map
// cache (the descriptors are encoded into stack storage).
//
// Limits and rules:
//  * B * S * Hq must not exceed YF_ATTN_NOALLOC_MAX_ROWS (32768 query rows x heads, e.g. one 2048-token
//    sequence with 16 heads); larger problems are refused with -3 and a message on stderr.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current).  Make that first call outside of any stream capture.
//  * All calls on a device share the one array and it keeps the previous call's contents; the part that must
//    start at zero (the dQ accumulator) is cleared by every call.  Two calls whose kernels overlap on the GPU
//    (different streams) race on it: keep calls on one device ordered.
//
// In host code the array's name is only a stand-in for the symbol, not a device address, so the host never
// passes it to a kernel: it passes the pointer that cudaGetSymbolAddress returned.
constexpr long long YF_ATTN_NOALLOC_MAX_ROWS = 32768;
constexpr long long NOALLOC_DELTA_FLOATS = YF_ATTN_NOALLOC_MAX_ROWS;                 // delta [B, Hq, S]
constexpr long long NOALLOC_DQ_FLOATS = YF_ATTN_NOALLOC_MAX_ROWS * 128;              // dQ accumulator [B*S, Hq*128]
static __device__ __align__(256) float g_attn_noalloc_scratch[NOALLOC_DELTA_FLOATS + NOALLOC_DQ_FLOATS];

static float* attn_noalloc_scratch_for_current_device(int* err) {
  static float* ptrs[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *err = e != cudaSuccess ? -(int)e : -1;
    return nullptr;
  }
  if (ptrs[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *err = e != cudaSuccess ? -(int)e : -1;
      return nullptr;
    }
    ptrs[dev] = p;
  }
  *err = 0;
  return ptrs[dev];
}

extern "C" int yf_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                                   void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, long long q_stride,
                                   long long kv_stride, long long o_stride, long long do_stride, long long dq_stride,
                                   long long dkv_stride, float scale, int causal, void* stream) {
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv)) return -1;
  if ((q_stride % 8) || (kv_stride % 8) || (o_stride % 8) || (do_stride % 8) || (dq_stride % 8) || (dkv_stride % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) |
       reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15)
    return -1;
  const long long rows = (long long)B * S * Hq;
  if (rows > YF_ATTN_NOALLOC_MAX_ROWS) {
    fprintf(stderr,
            "[yafsdp_b200] yf_attn_bwd_noalloc: B*S*Hq = %lld exceeds the built-in scratch for %lld rows; "
            "use yf_attn_bwd with caller-provided scratch\n",
            rows, YF_ATTN_NOALLOC_MAX_ROWS);
    return -3;
  }
  int err = 0;
  float* scratch = attn_noalloc_scratch_for_current_device(&err);
  if (scratch == nullptr) return err;
  float* delta = scratch;
  float* dq_accum = scratch + NOALLOC_DELTA_FLOATS;  // 131072 bytes in: still 256-byte aligned
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap mq, mk, mv, md, mdq;  // encoded in place: the cached variants would allocate a cache entry
  if (yf_tensor_map_3d_encode(&mq, q, (uint64_t)Hq * HD, S, B, q_stride, (uint64_t)S * q_stride, 64, BQ, 1, 2, 1) != 0 ||
      yf_tensor_map_3d_encode(&mk, k, (uint64_t)Hkv * HD, S, B, kv_stride, (uint64_t)S * kv_stride, 64, BKV, 1, 2, 1) != 0 ||
      yf_tensor_map_3d_encode(&mv, v, (uint64_t)Hkv * HD, S, B, kv_stride, (uint64_t)S * kv_stride, 64, BKV, 1, 2, 1) != 0 ||
      yf_tensor_map_3d_encode(&md, dout, (uint64_t)Hq * HD, S, B, do_stride, (uint64_t)S * do_stride, 64, BQ, 1, 2, 1) != 0 ||
      yf_tensor_map_3d_encode(&mdq, dq_accum, (uint64_t)Hq * HD, S, B, (uint64_t)Hq * HD, (uint64_t)S * Hq * HD, 32, BQ, 1, 4, 1) != 0)
    return -2;
  return attn_bwd_launch(mq, mk, mv, md, mdq, out, dout, lse, delta, dq_accum, dq, dk, dv, B, S, Hq, Hkv, o_stride, do_stride, dq_stride,
                         dkv_stride, scale, causal, st);
}
