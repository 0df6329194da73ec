// Causal flash-attention forward for head_dim 128 on sm_100a (MHA and GQA).
//
// One CTA per (128-row query tile, query head, sequence).  Roles:
//   warp 0     TMA producer: Q once, then K/V tiles of 128 keys through a 2-stage ring
//   warp 1     MMA issuer:   S = Q K^T (tcgen05, fp32 in TMEM, double-buffered) and O_j = P V
//   warps 2-9  softmax:      two threads per query row (TMEM lane == row; the pair splits the 128 key columns and
//                            the 128 output columns, and exchanges its partial row maximum through shared
//                            memory): online max / sum, P written as bf16 into 128-byte-swizzled shared memory
//                            (the A operand of the second MMA).
// The output accumulates in TMEM over all key blocks (O += P V).  The exponent's reference maximum is only moved when
// some row's maximum has grown by more than 2^8 since it was set (then every row rescales its O in TMEM and its sum);
// otherwise P is taken relative to the older maximum (values up to 2^8, harmless in bf16 / fp32), the softmax of block
// j+1 does not wait for the MMA of block j, and the final division by the row sum makes the result exact again.
// Inputs are read in place from the fused QKV projection output ([tokens, (Hq+2Hkv)*128], row pitch
// given), so no head transposes are materialised.  Writes O (bf16) and the log-sum-exp per row (fp32).
#include "common.cuh"
#include "yafsdp_b200.h"

YF_TU_STATUS()

namespace {

constexpr int HD = 128;        // head dim
constexpr int BQ = 128;        // query rows per CTA
constexpr int BKV = 128;       // keys per tile
constexpr int ATOM = 16384;    // bytes of one [128 rows x 64 bf16] swizzled block
constexpr int TILE = 2 * ATOM; // one 128x128 bf16 tile
constexpr int FWD_THREADS = 320;  // producer warp, MMA warp, eight softmax warps
constexpr int FWD_SMEM = 1024 + TILE /*Q*/ + 2 * 2 * TILE /*K,V x2 stages*/ + TILE /*P*/ + 256 + 3072 /*row max / sum exchange*/;

struct FwdArgs {
  __nv_bfloat16* out;
  float* lse;
  long long out_stride;  // elements between token rows of out
  int S, B, Hq, Hkv;
  float scale_log2;      // softmax scale * log2(e)
  float scale;
  int causal;
};

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, FwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + TILE;             // stage s: K at sKV + s*2*TILE, V at + TILE
  uint8_t* sP = sKV + 4 * TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + TILE);
  uint64_t* q_full = bars;              // 1
  uint64_t* k_full = bars + 1;          // 2
  uint64_t* v_full = bars + 3;          // 2
  uint64_t* kv_empty = bars + 5;        // 2
  uint64_t* s_full = bars + 7;          // 2
  uint64_t* p_ready = bars + 9;         // 1
  uint64_t* o_full = bars + 10;         // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  float* xmax = reinterpret_cast<float*>(bars + 32);   // [2 (block parity)][2 (column half)][128 rows]
  float* xsum = xmax + 512;                            // [2 (column half)][128 rows]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nq_tiles = gridDim.x;
  const int qt = args.causal ? (nq_tiles - 1 - blockIdx.x) : blockIdx.x;  // heavy tiles first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = h / (args.Hq / args.Hkv);
  const int q0 = qt * BQ;
  const int n_kv_total = (args.S + BKV - 1) / BKV;
  const int n_kv = args.causal ? min(qt + 1, n_kv_total) : n_kv_total;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(p_ready, 256);
    mbar_init(o_full, 1);
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
  const uint32_t tmem_S = tmem_base;          // two buffers of 128 columns
  const uint32_t tmem_O = tmem_base + 256;    // 128 columns

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE);
      tma_load_3d(sQ, &tma_q, q_full, h * HD, q0, b);
      tma_load_3d(sQ + ATOM, &tma_q, q_full, h * HD + 64, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, 100)) break;
        uint8_t* sK = sKV + s * 2 * TILE;
        uint8_t* sV = sK + TILE;
        mbar_expect_tx(&k_full[s], TILE);
        tma_load_3d(sK, &tma_k, &k_full[s], hkv * HD, j * BKV, b);
        tma_load_3d(sK + ATOM, &tma_k, &k_full[s], hkv * HD + 64, j * BKV, b);
        mbar_expect_tx(&v_full[s], TILE);
        tma_load_3d(sV, &tma_v, &v_full[s], hkv * HD, j * BKV, b);
        tma_load_3d(sV + ATOM, &tma_v, &v_full[s], hkv * HD + 64, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, 0, 0);   // Q, K both K-major (K = head dim)
      const uint32_t idesc_o = umma_idesc_bf16(BQ, HD, 0, 1);    // P K-major (K = keys), V MN-major
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      auto issue_s = [&](int j) {
        const uint32_t aK = smem_u32(sKV + (j & 1) * 2 * TILE);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * ATOM + (k & 3) * 32;
          tc_mma_bf16(tmem_S + (j & 1) * 128, umma_smem_desc_sw128(aQ + off, 0, 1024),
                      umma_smem_desc_sw128(aK + off, 0, 1024), idesc_s, k != 0);
        }
        tc_commit(&s_full[j & 1]);
      };
      bool alive = mbar_wait(q_full, 0, 110) && mbar_wait(&k_full[0], 0, 111);
      if (alive) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_kv && alive; ++j) {
        const int s = j & 1;
        if (j + 1 < n_kv) {
          if (!mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, 112)) { alive = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(p_ready, j & 1, 113) || !mbar_wait(&v_full[s], (j >> 1) & 1, 114)) { alive = false; break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(sKV + s * 2 * TILE + TILE);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          tc_mma_bf16(tmem_O, umma_smem_desc_sw128(aP + (k >> 2) * ATOM + (k & 3) * 32, 0, 1024),
                      umma_smem_desc_sw128(aV + k * 2048, ATOM, 1024), idesc_o, (j | k) != 0);  // O accumulates over the blocks
        }
        tc_commit(o_full);
        tc_commit(&kv_empty[s]);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;           // row inside the query tile == TMEM lane
    const int half = (warp - 2) >> 2;        // which 64 key columns / 64 output columns of the row this thread owns
    const int c_begin = half * 2;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;    // m_run: reference maximum of the exponent; l_run: this thread's half of the row sum
    const float sl2 = args.scale_log2;
    constexpr float RESCALE_LOG2 = 8.f;      // move the reference maximum when a row's maximum exceeds it by 2^8
    bool alive = true;
    bool gave_up = false;  // this thread's bounded wait ran out: all 256 softmax threads leave together at the next barrier
    for (int j = 0; j < n_kv && alive; ++j) {
      if (!gave_up && !mbar_wait(&s_full[j & 1], (j >> 1) & 1, 120)) gave_up = true;
      tc_fence_after();
      const uint32_t ts = tmem_S + lane_off + (j & 1) * 128;
      const int kv0 = j * BKV;
      // keys allowed for this row: col <= limit
      const int limit = args.causal ? min(q0 + row, args.S - 1) : (args.S - 1);
      const bool need_mask = (kv0 + BKV - 1 > limit);
      // this thread's 64 scores, read from TMEM once
      uint32_t sc[2][32];
      tmem_ld32(ts + c_begin * 32, sc[0]);
      tmem_ld32(ts + (c_begin + 1) * 32, sc[1]);
      tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          const bool ok = !need_mask || (kv0 + (c_begin + c) * 32 + t <= limit);
          if (ok) mx = fmaxf(mx, __uint_as_float(sc[c][t]));
        }
      }
      // combine with the partner thread's half (buffers alternate with the block parity: one barrier per block)
      float* xm = xmax + (j & 1) * 256;
      xm[half * 128 + row] = mx;
      if (named_bar_or(2, 256, gave_up)) { alive = false; break; }  // the barrier of the maximum exchange carries the give-up flag
      mx = fmaxf(mx, xm[(half ^ 1) * 128 + row]);
      // does any row of the tile need a new reference maximum?  (uniform over all softmax threads: they share TMEM loads)
      const bool grew = (j == 0) || (mx != -INFINITY && (m_run == -INFINITY || (mx - m_run) * sl2 > RESCALE_LOG2));
      if (named_bar_or(3, 256, grew)) {
        const float m_new = fmaxf(m_run, mx);
        if (j > 0) {
          // O holds sums relative to the old maximum: wait for the last P V to land, then scale this thread's 64 columns
          if (!mbar_wait(o_full, (j - 1) & 1, 121)) gave_up = true;
          tc_fence_after();
          const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * sl2);
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem_O + lane_off + (c_begin + c) * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 32; ++t) r[t] = __float_as_uint(__uint_as_float(r[t]) * alpha);
            tmem_st32(tmem_O + lane_off + (c_begin + c) * 32, r);
          }
          tmem_st_wait();
          l_run *= alpha;
        }
        m_run = m_new;
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      const float neg_ms = -m_use * sl2;
      float rowsum = 0.f;
      uint32_t packed[2][16];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(sc[c][t]), sl2, neg_ms));
          float p1 = fast_exp2(fmaf(__uint_as_float(sc[c][t + 1]), sl2, neg_ms));
          if (need_mask) {
            if (kv0 + (c_begin + c) * 32 + t > limit) p0 = 0.f;
            if (kv0 + (c_begin + c) * 32 + t + 1 > limit) p1 = 0.f;
          }
          rowsum += p0 + p1;
          packed[c][t >> 1] = pack_bf16x2(p0, p1);
        }
      }
      l_run += rowsum;
      // the P buffer is free once the previous block's P V has read it; by now that MMA has had the whole softmax to finish
      if (j > 0 && !mbar_wait(o_full, (j - 1) & 1, 122)) gave_up = true;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int cc = c_begin + c;
        uint8_t* prow = sP + (cc >> 1) * ATOM + row * 128;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int chunk = (cc & 1) * 4 + t;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[c][4 * t], packed[c][4 * t + 1], packed[c][4 * t + 2], packed[c][4 * t + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    // the output of the last block
    if (alive && n_kv > 0 && !mbar_wait(o_full, (n_kv - 1) & 1, 123)) gave_up = true;
    tc_fence_after();
    float o[HD / 2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_O + lane_off + (c_begin + c) * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int t = 0; t < 32; ++t) o[c * 32 + t] = __uint_as_float(r[t]);
    }
    // total row sum = both halves
    xsum[half * 128 + row] = l_run;
    if (named_bar_or(2, 256, gave_up)) alive = false;
    const float l_tot = l_run + xsum[(half ^ 1) * 128 + row];
    if (alive && q0 + row < args.S) {
      const float inv = (l_tot > 0.f) ? 1.f / l_tot : 0.f;
      __nv_bfloat16* dst = args.out + ((long long)b * args.S + q0 + row) * args.out_stride + h * HD + half * (HD / 2);
#pragma unroll
      for (int v = 0; v < HD / 16; ++v) {
        uint4 w;
        w.x = pack_bf16x2(o[8 * v + 0] * inv, o[8 * v + 1] * inv);
        w.y = pack_bf16x2(o[8 * v + 2] * inv, o[8 * v + 3] * inv);
        w.z = pack_bf16x2(o[8 * v + 4] * inv, o[8 * v + 5] * inv);
        w.w = pack_bf16x2(o[8 * v + 6] * inv, o[8 * v + 7] * inv);
        reinterpret_cast<uint4*>(dst)[v] = w;
      }
      if (half == 0)
        args.lse[((long long)b * args.Hq + h) * args.S + q0 + row] = (l_tot > 0.f) ? (m_run * args.scale + logf(l_tot)) : -INFINITY;
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

}  // namespace

// q, k, v: bf16 pointers to the first head's first column; token rows are q_stride / kv_stride elements
// apart (the three may alias one fused projection output).  Tokens are ordered [batch, seq].
// out: [B*S, out_stride] bf16 (head h at columns h*128), lse: [B, Hq, S] fp32.
extern "C" int yf_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Hq,
                           int Hkv, long long q_stride, long long kv_stride, long long out_stride, float scale, int causal,
                           void* stream) {
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv) || (q_stride % 8) || (kv_stride % 8) || (out_stride % 8)) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return -1;
  const CUtensorMap* mq = yf_tensor_map_3d(q, (uint64_t)Hq * HD, S, B, q_stride, (uint64_t)S * q_stride, 64, BQ, 1, 2, 1);
  const CUtensorMap* mk = yf_tensor_map_3d(k, (uint64_t)Hkv * HD, S, B, kv_stride, (uint64_t)S * kv_stride, 64, BKV, 1, 2, 1);
  const CUtensorMap* mv = yf_tensor_map_3d(v, (uint64_t)Hkv * HD, S, B, kv_stride, (uint64_t)S * kv_stride, 64, BKV, 1, 2, 1);
  if (!mq || !mk || !mv) return -2;
  static bool optin[64] = {};  // the shared-memory opt-in is a per-device attribute
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (!optin[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) return -(int)e;
    optin[dev] = true;
  }
  if (int rc = yf_tu_bind_status()) return rc;
  FwdArgs a;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.out_stride = out_stride;
  a.S = S; a.B = B; a.Hq = Hq; a.Hkv = Hkv;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.causal = causal ? 1 : 0;
  dim3 grid((S + BQ - 1) / BQ, Hq, B);
  attn_fwd_kernel<<<grid, FWD_THREADS, FWD_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(*mq, *mk, *mv, a);
  return -(int)cudaGetLastError();
}
