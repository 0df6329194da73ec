// Memory-bound kernels of the training step for sm_100a: RMSNorm, RoPE, SwiGLU, vocabulary
// cross-entropy, embedding, the sharded AdamW update fused with the bf16 all-gather-input refresh,
// gradient sum-of-squares, and flat casts.  All are 16-byte vectorised and sized to keep
// 148 SMs x several CTAs in flight; each is bandwidth-bound by design (one read and one write of
// every operand).
#include "common.cuh"
#include "yafsdp_b200.h"


namespace {

struct alignas(16) bf16x8 {
  uint32_t u[4];
};
YF_DEVINL void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
YF_DEVINL void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

template <int THREADS>
YF_DEVINL float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}
template <int THREADS>
YF_DEVINL float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : -INFINITY;
  t = warp_max(t);
  return t;
}

// ------------------------------------------------------------------ RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w ; one CTA per row, the row stays in registers between passes.
constexpr int RN_THREADS = 256;
constexpr int RN_MAXV = 4;  // vectors of 8 per thread held in registers: D <= 256*8*4 = 8192

__global__ void __launch_bounds__(RN_THREADS) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                                 int T, int D, float eps) {
  __shared__ float red[32];
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (size_t)row * D;
    float xv[RN_MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < RN_MAXV; ++i) {
      const int v = threadIdx.x + i * RN_THREADS;
      if (v < nvec) {
        load8(xr + v * 8, xv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += xv[i][j] * xv[i][j];
      }
    }
    for (int v = threadIdx.x + RN_MAXV * RN_THREADS; v < nvec; v += RN_THREADS) {  // rows wider than the register tile
      float t[8];
      load8(xr + v * 8, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += t[j] * t[j];
    }
    ss = block_sum<RN_THREADS>(ss, red);
    const float r = rsqrtf(ss / (float)D + eps);
    if (threadIdx.x == 0 && rstd) rstd[row] = r;
    __nv_bfloat16* yr = y + (size_t)row * D;
#pragma unroll
    for (int i = 0; i < RN_MAXV; ++i) {
      const int v = threadIdx.x + i * RN_THREADS;
      if (v < nvec) {
        float wv[8], o[8];
        load8(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = xv[i][j] * r * wv[j];
        store8(yr + v * 8, o);
      }
    }
    for (int v = threadIdx.x + RN_MAXV * RN_THREADS; v < nvec; v += RN_THREADS) {
      float t[8], wv[8], o[8];
      load8(xr + v * 8, t);
      load8(w + v * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = t[j] * r * wv[j];
      store8(yr + v * 8, o);
    }
  }
}

// Backward in two kernels.  (1) dx = r * (dy*w - xhat * mean(dy*w*xhat)) (+ dres, the gradient arriving
// through the residual branch, fused to save a pass): one CTA per row, the row stays in registers.
// (2) dw[j] += sum_rows dy * xhat: a column reduction over the token dimension, tiled [64 columns x a slice of
// rows] per CTA with one fp32 atomic per column per CTA.
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    const __nv_bfloat16* __restrict__ w,
                                                                    const __nv_bfloat16* __restrict__ dy,
                                                                    const float* __restrict__ rstd,
                                                                    const __nv_bfloat16* __restrict__ dres,
                                                                    __nv_bfloat16* __restrict__ dx, int T, int D) {
  __shared__ float red[32];
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (size_t)row * D;
    const __nv_bfloat16* dyr = dy + (size_t)row * D;
    const float r = rstd[row];
    float xh[RN_MAXV][8], g[RN_MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < RN_MAXV; ++i) {
      const int v = threadIdx.x + i * RN_THREADS;
      if (v < nvec) {
        float xv[8], dv[8], wv[8];
        load8(xr + v * 8, xv);
        load8(dyr + v * 8, dv);
        load8(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xv[j] * r;
          g[i][j] = dv[j] * wv[j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum<RN_THREADS>(dot, red) / (float)D;
    __nv_bfloat16* dxr = dx + (size_t)row * D;
#pragma unroll
    for (int i = 0; i < RN_MAXV; ++i) {
      const int v = threadIdx.x + i * RN_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (g[i][j] - xh[i][j] * dot);
        if (dres) {
          float e[8];
          load8(dres + (size_t)row * D + v * 8, e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        store8(dxr + v * 8, o);
      }
    }
  }
}

// G warps per row (G = 1, 2 or 4; D <= 32 * G * 8 * RNW_NV forward, RNW_NV_B backward), four warps per CTA: the row stays in registers as packed bf16,
// every operand of a row is requested before anything is reduced (one exposed memory latency per row, not one per pass),
// and the only synchronisation is a named barrier among the G warps of the row.  Thread t of a row's group holds the
// vectors t, t + 32 G, ... of the row (contiguous 512 G bytes per load instruction).
constexpr int RNW_WARPS = 4;
constexpr int RNW_NV = 8;    // forward: vectors of a row per thread
constexpr int RNW_NV_B = 4;  // backward (three operands per row in registers)
YF_DEVINL void unpack8(const uint4& v, float (&f)[8]) {
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <int G>
YF_DEVINL float row_group_sum(float v, float* red, int row_in_cta) {
  v = warp_sum(v);
  if (G == 1) return v;
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  if (row_in_cta == 0) named_bar_sync(1, 32 * G);  // literal barrier numbers: a computed one reserves all sixteen
  else named_bar_sync(2, 32 * G);
  float t = 0.f;
#pragma unroll
  for (int g = 0; g < G; ++g) t += red[row_in_cta * G + g];
  return t;
}

template <int G>
__global__ void __launch_bounds__(RNW_WARPS * 32) rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                                          const __nv_bfloat16* __restrict__ w,
                                                                          __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                                          int T, int D, float eps) {
  __shared__ float red[RNW_WARPS];
  constexpr int ROWS = RNW_WARPS / G, TPR = 32 * G;
  const int row_in_cta = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int row = blockIdx.x * ROWS + row_in_cta;
  if (row >= T) return;
  const int nvec = D / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 xv[RNW_NV], wv[RNW_NV];
#pragma unroll
  for (int i = 0; i < RNW_NV; ++i) {
    const int v = tr + TPR * i;
    xv[i] = v < nvec ? xr[v] : make_uint4(0u, 0u, 0u, 0u);
    wv[i] = v < nvec ? __ldg(wr + v) : make_uint4(0u, 0u, 0u, 0u);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < RNW_NV; ++i) {
    float f[8];
    unpack8(xv[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = row_group_sum<G>(ss, red, row_in_cta);
  const float r = rsqrtf(ss / (float)D + eps);
  if (tr == 0 && rstd) rstd[row] = r;
  __nv_bfloat16* yr = y + (size_t)row * D;
#pragma unroll
  for (int i = 0; i < RNW_NV; ++i) {
    const int v = tr + TPR * i;
    if (v < nvec) {
      float f[8], wf[8], o[8];
      unpack8(xv[i], f);
      unpack8(wv[i], wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = f[j] * r * wf[j];
      store8(yr + v * 8, o);
    }
  }
}

// dx of the same form; CTA 0 also clears the weight gradient when `dw_zero` is given (the column-reduction kernel that
// accumulates into it is launched after this one on the same stream).
template <int G>
__global__ void __launch_bounds__(RNW_WARPS * 32, 6) rmsnorm_bwd_dx_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                                                const __nv_bfloat16* __restrict__ w,
                                                                                const __nv_bfloat16* __restrict__ dy,
                                                                                const float* __restrict__ rstd,
                                                                                const __nv_bfloat16* __restrict__ dres,
                                                                                __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_zero,
                                                                                int T, int D) {
  __shared__ float red[RNW_WARPS];
  if (dw_zero != nullptr && blockIdx.x == 0)
    for (int i = threadIdx.x; i < D; i += RNW_WARPS * 32) dw_zero[i] = 0.f;
  constexpr int ROWS = RNW_WARPS / G, TPR = 32 * G;
  const int row_in_cta = threadIdx.x / TPR, tr = threadIdx.x % TPR;
  const int row = blockIdx.x * ROWS + row_in_cta;
  if (row >= T) return;
  const int nvec = D / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
  const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * D);
  const uint4* er = reinterpret_cast<const uint4*>(dres ? dres + (size_t)row * D : x);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 xv[RNW_NV_B], dv[RNW_NV_B], ev[RNW_NV_B];
#pragma unroll
  for (int i = 0; i < RNW_NV_B; ++i) {
    const int v = tr + TPR * i;
    const bool in = v < nvec;
    xv[i] = in ? xr[v] : make_uint4(0u, 0u, 0u, 0u);
    dv[i] = in ? dyr[v] : make_uint4(0u, 0u, 0u, 0u);
    ev[i] = (in && dres) ? er[v] : make_uint4(0u, 0u, 0u, 0u);
  }
  const float r = rstd[row];
  // g = dy * w replaces dy in registers (fp32 products rounded to bf16 would lose bits: keep dy and w apart instead and
  // multiply twice; w comes from L1 both times)
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < RNW_NV_B; ++i) {
    const int v = tr + TPR * i;
    if (v < nvec) {
      float xf[8], df[8], wf[8];
      unpack8(xv[i], xf);
      unpack8(dv[i], df);
      unpack8(__ldg(wr + v), wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += df[j] * wf[j] * (xf[j] * r);
    }
  }
  dot = row_group_sum<G>(dot, red, row_in_cta) / (float)D;
  __nv_bfloat16* dxr = dx + (size_t)row * D;
#pragma unroll
  for (int i = 0; i < RNW_NV_B; ++i) {
    const int v = tr + TPR * i;
    if (v < nvec) {
      float xf[8], df[8], wf[8], ef[8], o[8];
      unpack8(xv[i], xf);
      unpack8(dv[i], df);
      unpack8(ev[i], ef);
      unpack8(__ldg(wr + v), wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = r * (df[j] * wf[j] - xf[j] * r * dot) + ef[j];
      store8(dxr + v * 8, o);
    }
  }
}

constexpr int RN_DW_COLS = 64;     // columns per CTA (8 threads x 8 bf16)
constexpr int RN_DW_ROWLANES = 32; // row lanes per CTA (256 threads / 8)
__global__ void __launch_bounds__(256) rmsnorm_bwd_dw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                             const float* __restrict__ rstd, float* __restrict__ dw, int T, int D,
                                                             int rows_per_cta) {
  __shared__ float part[RN_DW_ROWLANES][RN_DW_COLS + 1];
  const int c8 = threadIdx.x & 7;
  const int rl = threadIdx.x >> 3;
  const int col = blockIdx.x * RN_DW_COLS + c8 * 8;
  const int row0 = blockIdx.y * rows_per_cta;
  const int row1 = min(T, row0 + rows_per_cta);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (col < D) {
    for (int row = row0 + rl; row < row1; row += RN_DW_ROWLANES) {
      float xv[8], dv[8];
      load8(x + (size_t)row * D + col, xv);
      load8(dy + (size_t)row * D + col, dv);
      const float r = rstd[row];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += dv[j] * xv[j] * r;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[rl][c8 * 8 + j] = acc[j];
  __syncthreads();
  if (threadIdx.x < RN_DW_COLS) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < RN_DW_ROWLANES; ++r) s += part[r][threadIdx.x];
    const int c = blockIdx.x * RN_DW_COLS + threadIdx.x;
    if (c < D) atomicAdd(dw + c, s);
  }
}

// ------------------------------------------------------------------ RoPE (rotate-half pairing, in place)
// qkv: [T, row_stride] bf16 with n_heads heads of head_dim starting at column col0; pos = row % seq_len.
// cos/sin table: [seq_len, head_dim/2] fp32.  sign = +1 forward, -1 backward (inverse rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cs, int T, int seq_len,
                            long long row_stride, int col0, int n_heads, int head_dim, float sign) {
  const int half = head_dim / 2;
  const int vec_per_head = half / 8;
  const long long total = (long long)T * n_heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    const long long th = i / vec_per_head;
    const int h = (int)(th % n_heads);
    const long long t = th / n_heads;
    const int pos = (int)(t % seq_len);
    __nv_bfloat16* p = qkv + t * row_stride + col0 + h * head_dim + v * 8;
    float a[8], b[8], oa[8], ob[8];
    load8(p, a);
    load8(p + half, b);
    const float* c = cs + ((size_t)pos * half + v * 8) * 2;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float co = c[2 * j], si = c[2 * j + 1] * sign;
      oa[j] = a[j] * co - b[j] * si;
      ob[j] = b[j] * co + a[j] * si;
    }
    store8(p, oa);
    store8(p + half, ob);
  }
}

// ------------------------------------------------------------------ SwiGLU
// gu: [T, 2F] (gate columns [0,F), up columns [F,2F)); h = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long T, int F) {
  const int vpr = F / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    float g[8], u[8], o[8];
    load8(gu + t * 2 * F + v * 8, g);
    load8(gu + t * 2 * F + F + v * 8, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(h + t * F + v * 8, o);
  }
}
// dgate = dh * up * (sig + g*sig*(1-sig)), dup = dh * silu(g); written into dgu [T, 2F]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int vpr = F / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    float g[8], u[8], d[8], og[8], ou[8];
    load8(gu + t * 2 * F + v * 8, g);
    load8(gu + t * 2 * F + F + v * 8, u);
    load8(dh + t * F + v * 8, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      og[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
      ou[j] = d[j] * g[j] * s;
    }
    store8(dgu + t * 2 * F + v * 8, og);
    store8(dgu + t * 2 * F + F + v * 8, ou);
  }
}

// ------------------------------------------------------------------ cross-entropy (forward + backward in one pass pair)
// logits [T, V] bf16 (row pitch ldl) are replaced in place by dlogits = (softmax - onehot) * grad_scale, where grad_scale is
// the host value times *scale_ptr when that device pointer is given (e.g. 1 / number of valid labels, counted on the device);
// loss_rows[t] = logsumexp - logit[label] (0 for ignored rows, label < 0).  One CTA per row.
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits,
                                                                   const long long* __restrict__ labels,
                                                                   float* __restrict__ loss_rows, int T, int V,
                                                                   long long ldl, float grad_scale,
                                                                   const float* __restrict__ scale_ptr, int write_grad) {
  __shared__ float red[32];
  const int nvec = V / 8;
  if (scale_ptr != nullptr) grad_scale *= *scale_ptr;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    __nv_bfloat16* lr = logits + (size_t)row * ldl;
    const long long label = labels[row];
    if (label < 0 || label >= V) {
      if (threadIdx.x == 0) loss_rows[row] = 0.f;
      if (write_grad) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int v = threadIdx.x; v < nvec; v += CE_THREADS) *reinterpret_cast<uint4*>(lr + v * 8) = z;
        for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) lr[j] = __float2bfloat16_rn(0.f);
      }
      continue;
    }
    // online max / sum-exp
    float m = -INFINITY, s = 0.f;
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      float f[8];
      load8(lr + v * 8, f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
      const float f = __bfloat162float(lr[j]);
      const float nm = fmaxf(m, f);
      s = s * __expf(m - nm) + __expf(f - nm);
      m = nm;
    }
    const float gm = block_max<CE_THREADS>(m, red);
    const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
    const float gs = block_sum<CE_THREADS>(contrib, red);
    const float lse = gm + __logf(gs);
    if (threadIdx.x == 0) loss_rows[row] = lse - __bfloat162float(lr[label]);
    if (write_grad) {
      __syncthreads();  // the label logit was read above before anyone overwrites it
      for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
        float f[8], o[8];
        load8(lr + v * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float p = __expf(f[j] - lse);
          if (v * 8 + j == label) p -= 1.f;
          o[j] = p * grad_scale;
        }
        store8(lr + v * 8, o);
      }
      for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
        float p = __expf(__bfloat162float(lr[j]) - lse);
        if (j == label) p -= 1.f;
        lr[j] = __float2bfloat16_rn(p * grad_scale);
      }
    }
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ ids,
                                     __nv_bfloat16* __restrict__ out, long long T, int D, int V) {
  const int vpr = D / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    long long id = ids[t];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < V) val = *reinterpret_cast<const uint4*>(table + id * D + v * 8);
    *reinterpret_cast<uint4*>(out + t * D + v * 8) = val;
  }
}
// dtable[ids[t], :] += dout[t, :]  (fp32 table gradient, atomics: token ids repeat)
__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ ids,
                                     float* __restrict__ dtable, long long T, int D, int V) {
  const int vpr = D / 8;
  const long long total = T * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpr;
    const int v = (int)(i % vpr);
    const long long id = ids[t];
    if (id < 0 || id >= V) continue;
    float f[8];
    load8(dout + t * D + v * 8, f);
    float* dst = dtable + id * D + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, f[j]);
  }
}

// ------------------------------------------------------------------ AdamW on the flat fp32 master shard
// p, m, v updated in place from g (scaled by *grad_scale_ptr when given, e.g. the clip coefficient);
// the bf16 copy that the next all-gather reads is refreshed in the same pass.
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^step
};
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                                    float* __restrict__ v, __nv_bfloat16* __restrict__ p_bf16,
                                                    const float* __restrict__ grad_scale_ptr, long long n, AdamArgs a) {
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  const float inv_bc1 = 1.f / a.bc1;
  const float inv_sqrt_bc2 = rsqrtf(a.bc2);
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float pe[4] = {pv.x, pv.y, pv.z, pv.w}, ge[4] = {gv.x, gv.y, gv.z, gv.w}, me[4] = {mv.x, mv.y, mv.z, mv.w},
          ve[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = ge[j] * gs;
      pe[j] *= (1.f - a.lr * a.weight_decay);
      me[j] = a.beta1 * me[j] + (1.f - a.beta1) * gr;
      ve[j] = a.beta2 * ve[j] + (1.f - a.beta2) * gr * gr;
      const float denom = sqrtf(ve[j]) * inv_sqrt_bc2 + a.eps;
      pe[j] -= a.lr * (me[j] * inv_bc1) / denom;
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pe[0], pe[1], pe[2], pe[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(me[0], me[1], me[2], me[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(ve[0], ve[1], ve[2], ve[3]);
    if (p_bf16) {
      uint2 o;
      o.x = pack_bf16x2(pe[0], pe[1]);
      o.y = pack_bf16x2(pe[2], pe[3]);
      reinterpret_cast<uint2*>(p_bf16)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  for (long long i = nvec * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gr = g[i] * gs;
    float pe = p[i] * (1.f - a.lr * a.weight_decay);
    const float me = a.beta1 * m[i] + (1.f - a.beta1) * gr;
    const float ve = a.beta2 * v[i] + (1.f - a.beta2) * gr * gr;
    pe -= a.lr * (me * inv_bc1) / (sqrtf(ve) * inv_sqrt_bc2 + a.eps);
    p[i] = pe; m[i] = me; v[i] = ve;
    if (p_bf16) p_bf16[i] = __float2bfloat16_rn(pe);
  }
}

// ------------------------------------------------------------------ sum of squares (gradient norm), fp32 -> *out += sum
__global__ void __launch_bounds__(256) sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = nvec * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    acc += g[i] * g[i];
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// clip coefficient from the total squared norm: coef = min(1, max_norm / (sqrt(total) + 1e-6)); norm_out = sqrt(total)
__global__ void clip_coef_kernel(const float* __restrict__ total_sq, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float nrm = sqrtf(*total_sq);
  if (norm_out) *norm_out = nrm;
  *coef = fminf(1.f, max_norm / (nrm + 1e-6f));
}

// ------------------------------------------------------------------ flat casts / scale
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(src)[2 * i], b = reinterpret_cast<const float4*>(src)[2 * i + 1];
    uint4 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    o.z = pack_bf16x2(b.x, b.y);
    o.w = pack_bf16x2(b.z, b.w);
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
  for (long long i = nvec * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}
// dst(fp32) = or += scale * src(bf16)
__global__ void accum_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n,
                                         float scale, int accumulate) {
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    load8(src + i * 8, f);
    float4 a = make_float4(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
    float4 b = make_float4(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
    if (accumulate) {
      const float4 oa = reinterpret_cast<float4*>(dst)[2 * i], ob = reinterpret_cast<float4*>(dst)[2 * i + 1];
      a.x += oa.x; a.y += oa.y; a.z += oa.z; a.w += oa.w;
      b.x += ob.x; b.y += ob.y; b.z += ob.z; b.w += ob.w;
    }
    reinterpret_cast<float4*>(dst)[2 * i] = a;
    reinterpret_cast<float4*>(dst)[2 * i + 1] = b;
  }
  for (long long i = nvec * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float f = __bfloat162float(src[i]) * scale;
    dst[i] = accumulate ? dst[i] + f : f;
  }
}
// y = a + b (bf16), used for residual joins in backward
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long long n) {
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float x[8], z[8], o[8];
    load8(a + i * 8, x);
    load8(b + i * 8, z);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = x[j] + z[j];
    store8(y + i * 8, o);
  }
  for (long long i = nvec * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16_rn(__bfloat162float(a[i]) + __bfloat162float(b[i]));
}

inline int grid_for(long long work_items, int threads, int ctas_per_sm) {
  long long need = (work_items + threads - 1) / threads;
  long long cap = (long long)yf_num_sms() * ctas_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

#define YF_STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define YF_LAUNCH_RET() return -(int)cudaGetLastError()

extern "C" int yf_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int T, int D, float eps, void* stream) {
  if (T <= 0 || D <= 0 || (D % 8) || !aligned16(x) || !aligned16(w) || !aligned16(y)) return -1;
  if (D <= 32 * 4 * 8 * RNW_NV) {  // G warps per row
    const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *wp = (const __nv_bfloat16*)w;
    __nv_bfloat16* yp = (__nv_bfloat16*)y;
    const int g = D <= 32 * 8 * RNW_NV ? 1 : (D <= 64 * 8 * RNW_NV ? 2 : 4);
    const int rows = RNW_WARPS / g, ctas = (T + rows - 1) / rows;
    if (g == 1) rmsnorm_fwd_warp_kernel<1><<<ctas, RNW_WARPS * 32, 0, YF_STREAM(stream)>>>(xp, wp, yp, rstd, T, D, eps);
    else if (g == 2) rmsnorm_fwd_warp_kernel<2><<<ctas, RNW_WARPS * 32, 0, YF_STREAM(stream)>>>(xp, wp, yp, rstd, T, D, eps);
    else rmsnorm_fwd_warp_kernel<4><<<ctas, RNW_WARPS * 32, 0, YF_STREAM(stream)>>>(xp, wp, yp, rstd, T, D, eps);
    YF_LAUNCH_RET();
  }
  const int grid = T < yf_num_sms() * 8 ? T : yf_num_sms() * 8;
  rmsnorm_fwd_kernel<<<grid, RN_THREADS, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                                 (__nv_bfloat16*)y, rstd, T, D, eps);
  YF_LAUNCH_RET();
}
extern "C" int yf_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                              float* dw, int zero_dw, int T, int D, void* stream) {
  if (T <= 0 || D <= 0 || (D % 8) || D > RN_THREADS * 8 * RN_MAXV) return -1;
  if (!aligned16(x) || !aligned16(w) || !aligned16(dy) || !aligned16(dx) || (dres && !aligned16(dres))) return -1;
  if (zero_dw && !dw) return -1;
  if (D <= 32 * 4 * 8 * RNW_NV_B) {  // G warps per row
    const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *wp = (const __nv_bfloat16*)w, *dyp = (const __nv_bfloat16*)dy,
                        *ep = (const __nv_bfloat16*)dres;
    __nv_bfloat16* dxp = (__nv_bfloat16*)dx;
    float* dwz = zero_dw ? dw : nullptr;
    const int g = D <= 32 * 8 * RNW_NV_B ? 1 : (D <= 64 * 8 * RNW_NV_B ? 2 : 4);
    const int rows = RNW_WARPS / g, ctas = (T + rows - 1) / rows;
    if (g == 1) rmsnorm_bwd_dx_warp_kernel<1><<<ctas, RNW_WARPS * 32, 0, YF_STREAM(stream)>>>(xp, wp, dyp, rstd, ep, dxp, dwz, T, D);
    else if (g == 2) rmsnorm_bwd_dx_warp_kernel<2><<<ctas, RNW_WARPS * 32, 0, YF_STREAM(stream)>>>(xp, wp, dyp, rstd, ep, dxp, dwz, T, D);
    else rmsnorm_bwd_dx_warp_kernel<4><<<ctas, RNW_WARPS * 32, 0, YF_STREAM(stream)>>>(xp, wp, dyp, rstd, ep, dxp, dwz, T, D);
  } else {
    if (zero_dw && cudaMemsetAsync(dw, 0, (size_t)D * sizeof(float), YF_STREAM(stream)) != cudaSuccess) return -2;
    const int grid = T < yf_num_sms() * 8 ? T : yf_num_sms() * 8;
    rmsnorm_bwd_dx_kernel<<<grid, RN_THREADS, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                                      (const __nv_bfloat16*)dy, rstd, (const __nv_bfloat16*)dres,
                                                                      (__nv_bfloat16*)dx, T, D);
  }
  if (dw) {
    const int col_blocks = (D + RN_DW_COLS - 1) / RN_DW_COLS;
    int splits = (yf_num_sms() * 6 + col_blocks - 1) / col_blocks;  // about six CTAs per SM in total
    const int max_splits = (T + RN_DW_ROWLANES - 1) / RN_DW_ROWLANES;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    const int rows_per_cta = (T + splits - 1) / splits;
    dim3 g2(col_blocks, (T + rows_per_cta - 1) / rows_per_cta);
    rmsnorm_bwd_dw_kernel<<<g2, 256, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, rstd, dw, T, D,
                                                             rows_per_cta);
  }
  YF_LAUNCH_RET();
}
extern "C" int yf_rope(void* qkv, const float* cos_sin, int T, int seq_len, long long row_stride, int col0, int n_heads,
                       int head_dim, int backward, void* stream) {
  if (T <= 0 || n_heads <= 0 || (head_dim % 16) || (row_stride % 8) || (col0 % 8) || !aligned16(qkv)) return -1;
  const long long items = (long long)T * n_heads * (head_dim / 16);
  rope_kernel<<<grid_for(items, 256, 8), 256, 0, YF_STREAM(stream)>>>((__nv_bfloat16*)qkv, cos_sin, T, seq_len, row_stride, col0,
                                                                       n_heads, head_dim, backward ? -1.f : 1.f);
  YF_LAUNCH_RET();
}
extern "C" int yf_swiglu_fwd(const void* gu, void* h, long long T, int F, void* stream) {
  if (T <= 0 || F <= 0 || (F % 8) || !aligned16(gu) || !aligned16(h)) return -1;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256, 8), 256, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)h, T, F);
  YF_LAUNCH_RET();
}
extern "C" int yf_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long T, int F, void* stream) {
  if (T <= 0 || F <= 0 || (F % 8) || !aligned16(gu) || !aligned16(dh) || !aligned16(dgu)) return -1;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256, 8), 256, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dh,
                                                                                   (__nv_bfloat16*)dgu, T, F);
  YF_LAUNCH_RET();
}
extern "C" int yf_cross_entropy(void* logits, const long long* labels, float* loss_rows, int T, int V, long long ldl,
                                float grad_scale, const float* scale_ptr, int write_grad, void* stream) {
  if (T <= 0 || V <= 0 || (ldl % 8) || !aligned16(logits)) return -1;
  const int grid = T < yf_num_sms() * 4 ? T : yf_num_sms() * 4;
  cross_entropy_kernel<<<grid, CE_THREADS, 0, YF_STREAM(stream)>>>((__nv_bfloat16*)logits, labels, loss_rows, T, V, ldl, grad_scale,
                                                                   scale_ptr, write_grad);
  YF_LAUNCH_RET();
}
extern "C" int yf_embedding_fwd(const void* table, const long long* ids, void* out, long long T, int D, int V, void* stream) {
  if (T <= 0 || (D % 8) || !aligned16(table) || !aligned16(out)) return -1;
  embedding_fwd_kernel<<<grid_for(T * (D / 8), 256, 8), 256, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)table, ids,
                                                                                      (__nv_bfloat16*)out, T, D, V);
  YF_LAUNCH_RET();
}
extern "C" int yf_embedding_bwd(const void* dout, const long long* ids, float* dtable, long long T, int D, int V, void* stream) {
  if (T <= 0 || (D % 8) || !aligned16(dout)) return -1;
  embedding_bwd_kernel<<<grid_for(T * (D / 8), 256, 8), 256, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)dout, ids, dtable, T, D, V);
  YF_LAUNCH_RET();
}
extern "C" int yf_adamw(float* p, const float* g, float* m, float* v, void* p_bf16, const float* grad_scale_ptr, long long n,
                        float lr, float beta1, float beta2, float eps, float weight_decay, int step, int max_ctas, void* stream) {
  if (n <= 0) return 0;
  if (!aligned16(p) || !aligned16(g) || !aligned16(m) || !aligned16(v) || (p_bf16 && (reinterpret_cast<uintptr_t>(p_bf16) & 7)))
    return -1;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  // max_ctas > 0 caps the grid: when the update runs beside GEMMs on another stream, three CTAs per SM leave the
  // thread slots and registers that a persistent GEMM CTA needs and still keep HBM saturated
  int grid = grid_for(n / 4 + 1, 256, 8);
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  adamw_kernel<<<grid, 256, 0, YF_STREAM(stream)>>>(p, g, m, v, (__nv_bfloat16*)p_bf16, grad_scale_ptr, n, a);
  YF_LAUNCH_RET();
}
extern "C" int yf_sumsq(const float* g, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  if (!aligned16(g)) return -1;
  sumsq_kernel<<<grid_for(n / 4 + 1, 256, 4), 256, 0, YF_STREAM(stream)>>>(g, n, out);
  YF_LAUNCH_RET();
}
extern "C" int yf_clip_coef(const float* total_sq, float max_norm, float* coef, float* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, YF_STREAM(stream)>>>(total_sq, max_norm, coef, norm_out);
  YF_LAUNCH_RET();
}
extern "C" int yf_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  if (!aligned16(src) || !aligned16(dst)) return -1;
  cast_f32_to_bf16_kernel<<<grid_for(n / 8 + 1, 256, 8), 256, 0, YF_STREAM(stream)>>>(src, (__nv_bfloat16*)dst, n);
  YF_LAUNCH_RET();
}
extern "C" int yf_accum_bf16_to_f32(const void* src, float* dst, long long n, float scale, int accumulate, void* stream) {
  if (n <= 0) return 0;
  if (!aligned16(src) || !aligned16(dst)) return -1;
  accum_bf16_to_f32_kernel<<<grid_for(n / 8 + 1, 256, 8), 256, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)src, dst, n, scale, accumulate);
  YF_LAUNCH_RET();
}
extern "C" int yf_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  if (!aligned16(a) || !aligned16(b) || !aligned16(y)) return -1;
  add_bf16_kernel<<<grid_for(n / 8 + 1, 256, 8), 256, 0, YF_STREAM(stream)>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                               (__nv_bfloat16*)y, n);
  YF_LAUNCH_RET();
}
