// Row kernels of the gated parallel block and the latent attention: RMSNorm in groups, short causal convolution with
// carried state, gated sum of sublayer terms, norm + rotation + paged write of a latent cache entry, rotation of the
// rotated part of every query head, token-id selection, scaling. One block per token row unless said otherwise. All
// arithmetic is 32-bit; every sum has an order fixed by the row's own sizes.
#include "common.cuh"
#include <math.h>

namespace {
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// ------------------------------------------------------------------------------------------------ add + grouped RMSNorm
// As add_rmsnorm (rows == nullptr: x += delta in place; else row selection), with the row split into G equal
// consecutive parts, each scaled by its own 1 / sqrt(mean(part^2) + eps). The block's 256 threads form teams of TEAM
// threads (a power of two, at least a warp); team t sums the parts t, t + teams, ...: a part's sum is a fixed chain per
// thread, the warp's butterfly, and the team's warps added in rising order, whatever else is in the step.
template <typename TW, typename TH>
__global__ void __launch_bounds__(256)
add_rmsnorm_groups_kernel(float* __restrict__ x, const float* __restrict__ delta, const TW* __restrict__ w,
                          TH* __restrict__ h, const int* __restrict__ rows, int n_src, int D, int G, int team, float eps,
                          int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float warp_ss[8];
  const int r = blockIdx.x;
  int src = r;
  TH* hr = h + (size_t)r * D;
  if (rows != nullptr) {
    src = rows[r];
    if (src < 0 || src >= n_src) {
      if (src >= n_src && threadIdx.x == 0) atomicOr(err, FZ_ERR_ROW_RANGE);
      for (int d = threadIdx.x; d < D; d += blockDim.x) hr[d] = Cvt<TH>::from_f(0.f);
      return;
    }
  }
  float* __restrict__ xr = x + (size_t)src * D;
  const float* __restrict__ dr = delta ? delta + (size_t)src * D : nullptr;
  const bool write_x = rows == nullptr && dr != nullptr;
  const int Dg = D / G;
  const int teams = blockDim.x / team, t = threadIdx.x / team, lt = threadIdx.x - t * team;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpt = team >> 5;     // warps per team
  constexpr int KEEP = 8;                        // values a thread keeps in registers between the two passes
  const bool keep = Dg <= KEEP * team;           // (else the second pass reads the row again)
  for (int g0 = 0; g0 < G; g0 += teams) {       // the same trip count for every thread: the barriers below are safe
    const int g = g0 + t;
    const int end = (g + 1) * Dg;
    float ss = 0.f;
    float v[KEEP];
    if (g < G && keep) {
#pragma unroll
      for (int i = 0; i < KEEP; ++i) {
        const int d = g * Dg + lt + i * team;
        v[i] = d < end ? xr[d] : 0.f;
      }
      if (dr) {
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
          const int d = g * Dg + lt + i * team;
          if (d < end) v[i] += dr[d];
        }
      }
#pragma unroll
      for (int i = 0; i < KEEP; ++i) {
        const int d = g * Dg + lt + i * team;
        if (write_x && d < end) xr[d] = v[i];
        ss = fmaf(v[i], v[i], ss);
      }
    } else if (g < G) {
#pragma unroll 4
      for (int d = g * Dg + lt; d < end; d += team) {
        float u = xr[d];
        if (dr) u += dr[d];
        if (write_x) xr[d] = u;
        ss = fmaf(u, u, ss);
      }
    }
    ss = warp_sum(ss);
    __syncthreads();
    if (lane == 0) warp_ss[warp] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < wpt; ++i) total += warp_ss[t * wpt + i];
    const float scale = 1.0f / sqrtf(total * (1.0f / (float)Dg) + eps);
    if (g < G && keep) {
#pragma unroll
      for (int i = 0; i < KEEP; ++i) {
        const int d = g * Dg + lt + i * team;
        if (d < end) hr[d] = Cvt<TH>::from_f(Cvt<TW>::to_f(w[d]) * (v[i] * scale));
      }
    } else if (g < G) {
#pragma unroll 4
      for (int d = g * Dg + lt; d < end; d += team) {
        float u = xr[d];
        if (dr && !write_x) u += dr[d];
        hr[d] = Cvt<TH>::from_f(Cvt<TW>::to_f(w[d]) * (u * scale));
      }
    }
  }
}

// The same for parts whose length is a multiple of 4 and at most 8 * team: a thread keeps two float4 groups of its part
// in registers (16-byte loads of x, delta and the weights, 16- or 8-byte stores of h), so the row is read once.
__device__ __forceinline__ float4 ld4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 u = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&u.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* d, float4 v) { *(float4*)d = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* d, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  *(uint2*)d = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
}

template <typename TW, typename TH>
__global__ void __launch_bounds__(256)
add_rmsnorm_groups_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, const TW* __restrict__ w,
                              TH* __restrict__ h, const int* __restrict__ rows, int n_src, int D, int G, int team,
                              float eps, int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float warp_ss[8];
  const int r = blockIdx.x;
  int src = r;
  TH* hr = h + (size_t)r * D;
  if (rows != nullptr) {
    src = rows[r];
    if (src < 0 || src >= n_src) {
      if (src >= n_src && threadIdx.x == 0) atomicOr(err, FZ_ERR_ROW_RANGE);
      for (int d = threadIdx.x; d < D; d += blockDim.x) hr[d] = Cvt<TH>::from_f(0.f);
      return;
    }
  }
  float* __restrict__ xr = x + (size_t)src * D;
  const float* __restrict__ dr = delta ? delta + (size_t)src * D : nullptr;
  const bool write_x = rows == nullptr && dr != nullptr;
  const int Dg = D / G;
  const int teams = blockDim.x / team, t = threadIdx.x / team, lt = threadIdx.x - t * team;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpt = team >> 5;
  for (int g0 = 0; g0 < G; g0 += teams) {
    const int g = g0 + t;
    const int d0 = g * Dg + 4 * lt, d1 = d0 + 4 * team, end = (g + 1) * Dg;
    const bool in0 = g < G && d0 < end, in1 = g < G && d1 < end;
    float4 v0 = in0 ? ld4(xr + d0) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 v1 = in1 ? ld4(xr + d1) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (dr) {
      const float4 e0 = in0 ? ld4(dr + d0) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 e1 = in1 ? ld4(dr + d1) : make_float4(0.f, 0.f, 0.f, 0.f);
      v0.x += e0.x; v0.y += e0.y; v0.z += e0.z; v0.w += e0.w;
      v1.x += e1.x; v1.y += e1.y; v1.z += e1.z; v1.w += e1.w;
      if (write_x) {
        if (in0) st4(xr + d0, v0);
        if (in1) st4(xr + d1, v1);
      }
    }
    float ss = 0.f;
    ss = fmaf(v0.x, v0.x, ss); ss = fmaf(v0.y, v0.y, ss); ss = fmaf(v0.z, v0.z, ss); ss = fmaf(v0.w, v0.w, ss);
    ss = fmaf(v1.x, v1.x, ss); ss = fmaf(v1.y, v1.y, ss); ss = fmaf(v1.z, v1.z, ss); ss = fmaf(v1.w, v1.w, ss);
    ss = warp_sum(ss);
    __syncthreads();
    if (lane == 0) warp_ss[warp] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < wpt; ++i) total += warp_ss[t * wpt + i];
    const float scale = 1.0f / sqrtf(total * (1.0f / (float)Dg) + eps);
    if (in0) {
      const float4 g4 = ld4(w + d0);
      st4(hr + d0, make_float4(g4.x * (v0.x * scale), g4.y * (v0.y * scale), g4.z * (v0.z * scale), g4.w * (v0.w * scale)));
    }
    if (in1) {
      const float4 g4 = ld4(w + d1);
      st4(hr + d1, make_float4(g4.x * (v1.x * scale), g4.y * (v1.y * scale), g4.z * (v1.z * scale), g4.w * (v1.w * scale)));
    }
  }
}

// ------------------------------------------------------------------------------------------------ short convolution
// seg: (first row, rows, first position, state slot) per portion. state: (slots, taps - 1, C) float32, oldest first.
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_kernel(const T* __restrict__ h, const T* __restrict__ w, const float* __restrict__ state,
                  const int* __restrict__ seg, const int* __restrict__ seq_row, T* __restrict__ out, int C, int taps,
                  int residual, int act, const float* __restrict__ bias) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const int s = seq_row[n];
  T* orow = out + (size_t)n * C;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;      // a thread per channel: grid (rows, channel blocks)
  if (c >= C) return;
  if (s < 0) {
    orow[c] = Cvt<T>::from_f(0.f);
    return;
  }
  const int row0 = seg[4 * s], slot = seg[4 * s + 3];
  const int i = n - row0;
  const float* st = state != nullptr && slot >= 0 ? state + (size_t)slot * (taps - 1) * C : nullptr;
  {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int k = i - (taps - 1) + j;
      float v = 0.f;
      if (k >= 0) v = Cvt<T>::to_f(h[(size_t)(row0 + k) * C + c]);
      else if (st != nullptr) v = st[(size_t)(taps - 1 + k) * C + c];
      acc = fmaf(Cvt<T>::to_f(w[(size_t)c * taps + j]), v, acc);
    }
    if (bias != nullptr) acc += bias[c];
    if (residual) acc += Cvt<T>::to_f(h[(size_t)n * C + c]);
    if (act) acc = acc * (1.0f / (1.0f + expf(-acc)));      // silu of the 32-bit sum
    orow[c] = Cvt<T>::from_f(acc);
  }
}

// The same with eight channels per thread (16-byte loads of the inputs, the state and the output) for C % 8 == 0.
__device__ __forceinline__ void ld8(const float* p, float* v) {
  const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *(const uint4*)p;
  const __nv_bfloat162* q = (const __nv_bfloat162*)&u;
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(q[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void st8(float* p, const float* v) {
  *(float4*)p = make_float4(v[0], v[1], v[2], v[3]);
  *(float4*)(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float* v) {
  uint4 u;
  __nv_bfloat162* q = (__nv_bfloat162*)&u;
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *(uint4*)p = u;
}

// TAPS > 0: the tap count is known at compile time and the thread's 8 x TAPS weights (contiguous in the (C, taps)
// matrix) come in as TAPS 16-byte groups (bfloat16) instead of one by one; TAPS == 0: any tap count.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128)
short_conv_vec_kernel(const T* __restrict__ h, const T* __restrict__ w, const float* __restrict__ state,
                      const int* __restrict__ seg, const int* __restrict__ seq_row, T* __restrict__ out, int C, int taps,
                      int residual, int act, const float* __restrict__ bias) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int s = seq_row[n];
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (s >= 0) {
    const int row0 = seg[4 * s], slot = seg[4 * s + 3];
    const int i = n - row0;
    const float* st = state != nullptr && slot >= 0 ? state + (size_t)slot * (taps - 1) * C : nullptr;
    if constexpr (TAPS > 0) {
      float wv[8 * TAPS];                  // wv[e * TAPS + j]: tap j of channel c0 + e
#pragma unroll
      for (int m = 0; m < TAPS; ++m) ld8(w + (size_t)c0 * TAPS + 8 * m, wv + 8 * m);
#pragma unroll
      for (int j = 0; j < TAPS; ++j) {
        const int k = i - (TAPS - 1) + j;
        float v[8];
        if (k >= 0) ld8(h + (size_t)(row0 + k) * C + c0, v);
        else if (st != nullptr) ld8(st + (size_t)(TAPS - 1 + k) * C + c0, v);
        else continue;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wv[e * TAPS + j], v[e], acc[e]);
      }
    } else {
      for (int j = 0; j < taps; ++j) {
        const int k = i - (taps - 1) + j;
        float v[8];
        if (k >= 0) ld8(h + (size_t)(row0 + k) * C + c0, v);
        else if (st != nullptr) ld8(st + (size_t)(taps - 1 + k) * C + c0, v);
        else continue;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(Cvt<T>::to_f(w[(size_t)(c0 + e) * taps + j]), v[e], acc[e]);
      }
    }
    if (bias != nullptr) {
      float v[8];
      ld8(bias + c0, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
    if (residual) {
      float v[8];
      ld8(h + (size_t)n * C + c0, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += v[e];
    }
    if (act) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = acc[e] * (1.0f / (1.0f + expf(-acc[e])));      // silu of the 32-bit sum
    }
  }
  st8(out + (size_t)n * C + c0, acc);
}

// After the convolution has read the old state: the state of every portion's request becomes its last taps - 1 inputs
// (the portion's own rows, and what is left of the old state when the portion is shorter than taps - 1). A thread owns
// one channel of one portion, reads all it needs and then writes. grid (portions, channel blocks).
constexpr int MAX_TAPS = 32;
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const T* __restrict__ h, float* __restrict__ state, const int* __restrict__ seg, int C, int taps) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], slot = seg[4 * s + 3];
  if (c >= C || cnt <= 0 || slot < 0) return;
  float* st = state + (size_t)slot * (taps - 1) * C;
  float keep[MAX_TAPS - 1];
#pragma unroll
  for (int m = 0; m < MAX_TAPS - 1; ++m) {
    if (m < taps - 1) {
      const int k = cnt - (taps - 1) + m;
      keep[m] = k >= 0 ? Cvt<T>::to_f(h[(size_t)(row0 + k) * C + c]) : st[(size_t)(taps - 1 + k) * C + c];
    }
  }
#pragma unroll
  for (int m = 0; m < MAX_TAPS - 1; ++m)
    if (m < taps - 1) st[(size_t)m * C + c] = keep[m];
}

// ------------------------------------------------------------------------------------------------ gated sum
// out = a * sigmoid(ga) + (fw * sum_k f[n * terms + k]) * sigmoid(gf); a null gate counts as 1, f null as no term.
__global__ void gated_sum_kernel(const float* __restrict__ a, const float* __restrict__ ga, const float* __restrict__ f,
                                 const float* __restrict__ gf, float* __restrict__ out, int N, int D, int terms, float fw) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const size_t total = (size_t)N * D;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const size_t n = e / D, d = e - n * D;
    float y = a[e];
    if (ga) y *= sigmoidf_(ga[e]);
    if (f) {
      float t = 0.f;
      for (int k = 0; k < terms; ++k) t += f[(n * terms + k) * D + d];
      t *= fw;
      if (gf) t *= sigmoidf_(gf[e]);
      y += t;
    }
    out[e] = y;
  }
}

__global__ void scale_kernel(float* __restrict__ x, float factor, size_t total) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x)
    x[e] = x[e] * factor;
}

__global__ void select_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ src,
                                     const int* __restrict__ prev_ids, int* __restrict__ out, int N) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n < N) out[n] = src[n] >= 0 ? prev_ids[src[n]] : tokens[n];
}

// Which dimension d of a rotated vector is turned with, the pair's index in the tables, and whether d is the pair's first
// member. pairing 0: d with d + half; 1: 2i with 2i + 1.
__device__ __forceinline__ void rot_pair_of(int d, int half, int pairing, int& partner, int& pair, bool& first) {
  if (pairing == 0) { first = d < half; partner = first ? d + half : d - half; pair = first ? d : d - half; }
  else { first = (d & 1) == 0; partner = d ^ 1; pair = d >> 1; }
}

// ------------------------------------------------------------------------------------------------ latent cache entry
// down: (N, L + R) float32. The row's cache entry = [w * down[:L] / rms(down[:L]) | turn(down[L:])], rounded once, stored
// at the row's place in its pages. pool: (pages, page_size, L + R).
template <typename TW, typename T>
__global__ void __launch_bounds__(256)
latent_cache_write_kernel(const float* __restrict__ down, const TW* __restrict__ w, float eps,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rotated,
                          const int* __restrict__ pos, const int* __restrict__ seq_row, const int* __restrict__ table,
                          int mb, T* __restrict__ pool, long long page_stride, int page_size, int L, int R, int max_len,
                          int num_pages, int* err, int pairing) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float scratch[32];
  const int n = blockIdx.x;
  const int row = seq_row[n];
  if (row < 0) return;
  const int p = pos[n];
  if (p < 0 || p >= max_len) {
    if (threadIdx.x == 0) atomicOr(err, FZ_ERR_POS_RANGE);
    return;
  }
  const int page = table[(size_t)row * mb + p / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, FZ_ERR_NO_PAGE);
    return;
  }
  const float* in = down + (size_t)n * (L + R);
  T* e = pool + (size_t)page * page_stride + (size_t)(p % page_size) * (L + R);
  float ss = 0.f;
  for (int d = threadIdx.x; d < L; d += blockDim.x) ss = fmaf(in[d], in[d], ss);
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss * (1.0f / (float)L) + eps);
  for (int d = threadIdx.x; d < L; d += blockDim.x) e[d] = Cvt<T>::from_f(Cvt<TW>::to_f(w[d]) * (in[d] * scale));
  const int half = rotated >> 1;
  const float* cr = cos_t + (size_t)p * half;
  const float* sr = sin_t + (size_t)p * half;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float v = in[L + d];
    if (d < rotated) {
      int partner, pair;
      bool first;
      rot_pair_of(d, half, pairing, partner, pair, first);
      const float other = in[L + partner];
      float o1, o2;
      fz_rope_pair(first ? v : other, first ? other : v, cr[pair], sr[pair], o1, o2);
      v = first ? o1 : o2;
    }
    e[L + d] = Cvt<T>::from_f(v);
  }
}

// ------------------------------------------------------------------------------------------------ rotation of heads
// q: (N, H, W); out[n, h, out_off + d] = turn(q[n, h, off + d]) for d < W - off. grid (N), threads over (h, d).
template <typename T>
__global__ void __launch_bounds__(256)
rotate_heads_kernel(const T* __restrict__ q, int W, int off, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, int rotated, const int* __restrict__ pos,
                    const int* __restrict__ seq_row, T* __restrict__ out, int Wo, int out_off, int H, int max_len, int* err,
                    int pairing) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const int R = W - off, half = rotated >> 1;
  const int p = pos[n];
  const bool live = seq_row[n] >= 0 && p >= 0 && p < max_len;
  if (seq_row[n] >= 0 && !live && threadIdx.x == 0) atomicOr(err, FZ_ERR_POS_RANGE);
  const float* cr = cos_t + (size_t)(live ? p : 0) * half;
  const float* sr = sin_t + (size_t)(live ? p : 0) * half;
  for (int e = threadIdx.x; e < H * R; e += blockDim.x) {
    const int hh = e / R, d = e - hh * R;
    const T* in = q + ((size_t)n * H + hh) * W + off;
    float v = 0.f;
    if (live) {
      v = Cvt<T>::to_f(in[d]);
      if (d < rotated) {
        int partner, pair;
        bool first;
        rot_pair_of(d, half, pairing, partner, pair, first);
        const float other = Cvt<T>::to_f(in[partner]);
        float o1, o2;
        fz_rope_pair(first ? v : other, first ? other : v, cr[pair], sr[pair], o1, o2);
        v = first ? o1 : o2;
      }
    }
    out[((size_t)n * H + hh) * Wo + out_off + d] = Cvt<T>::from_f(v);
  }
}
template <typename T>
void launch_conv_vec(dim3 grid, cudaStream_t stream, const T* h, const T* w, const float* state, const int* seg,
                     const int* seq_row, T* out, int C, int taps, int residual, int act, const float* bias) {
  const bool w_ok = ((uintptr_t)w & 15) == 0;       // the grouped weight loads want 16-byte aligned rows of 8 x taps values
#define FZ_CV(N) fz_launch(short_conv_vec_kernel<T, N>, grid, dim3(128), 0, stream, h, w, state, seg, seq_row, out, C, taps, residual, act, bias)
  if (w_ok && taps == 2) FZ_CV(2);
  else if (w_ok && taps == 3) FZ_CV(3);
  else if (w_ok && taps == 4) FZ_CV(4);
  else if (w_ok && taps == 5) FZ_CV(5);
  else if (w_ok && taps == 8) FZ_CV(8);
  else FZ_CV(0);
#undef FZ_CV
}
}  // namespace

FZ_API int fz_add_rmsnorm_groups(float* x, const float* delta, const void* w, int w_dtype, void* h, int h_dtype,
                                 const int* rows, int n_out, int n_src, int D, int G, float eps, int* err,
                                 cudaStream_t stream) {
  if (n_out <= 0) return FZ_OK;
  if (G <= 0 || D % G) return FZ_BAD_SHAPE;
  // teams of 256, 128, 64 or 32 threads: the largest that still gives every part a team in one pass, but no more
  // threads than a part has values
  int team = 256;
  while (team > 32 && (256 / team < G || team > D / G)) team >>= 1;
  // the vectorised kernel: parts of a multiple of 4 values, at most 8 per thread of the team, everything 16-byte aligned
  const bool vec = (D / G) % 4 == 0 && D / G <= 8 * team && (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)h) & 15) == 0;
#define FZ_GN(TW, TH) do { \
    if (vec) fz_launch(add_rmsnorm_groups_vec_kernel<TW, TH>, dim3(n_out), dim3(256), 0, stream, x, delta, (const TW*)w, (TH*)h, rows, n_src, D, G, team, eps, err); \
    else fz_launch(add_rmsnorm_groups_kernel<TW, TH>, dim3(n_out), dim3(256), 0, stream, x, delta, (const TW*)w, (TH*)h, rows, n_src, D, G, team, eps, err); \
    FZ_LAUNCH_CHECK(); return FZ_OK; } while (0)
  if (w_dtype == FZ_F32 && h_dtype == FZ_F32) FZ_GN(float, float);
  if (w_dtype == FZ_F32 && h_dtype == FZ_BF16) FZ_GN(float, __nv_bfloat16);
  if (w_dtype == FZ_BF16 && h_dtype == FZ_BF16) FZ_GN(__nv_bfloat16, __nv_bfloat16);
  if (w_dtype == FZ_BF16 && h_dtype == FZ_F32) FZ_GN(__nv_bfloat16, float);
#undef FZ_GN
  return FZ_BAD_DTYPE;
}

FZ_API int fz_short_conv(const void* h, const void* w, float* state, const int* seg, const int* seq_row, void* out,
                         int dtype, int N, int n_seg, int C, int taps, int residual, int act, const float* bias,
                         cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (taps < 1 || taps > MAX_TAPS) return FZ_BAD_SHAPE;
  const bool vec = C % 8 == 0 && (((uintptr_t)h | (uintptr_t)out | (uintptr_t)state | (uintptr_t)bias) & 15) == 0;
  const dim3 vgrid(N, (C / 8 + 127) / 128);
  if (dtype == FZ_F32) {
    if (vec) launch_conv_vec<float>(vgrid, stream, (const float*)h, (const float*)w, (const float*)state, seg, seq_row, (float*)out, C, taps, residual, act, bias);
    else fz_launch(short_conv_kernel<float>, dim3(N, (C + 255) / 256), dim3(256), 0, stream, (const float*)h, (const float*)w, (const float*)state, seg, seq_row, (float*)out, C, taps, residual, act, bias);
    FZ_LAUNCH_CHECK();
    if (taps > 1 && state != nullptr && n_seg > 0)
      fz_launch(short_conv_state_kernel<float>, dim3(n_seg, (C + 255) / 256), dim3(256), 0, stream, (const float*)h, state, seg, C, taps);
  } else if (dtype == FZ_BF16) {
    if (vec) launch_conv_vec<__nv_bfloat16>(vgrid, stream, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, (const float*)state, seg, seq_row, (__nv_bfloat16*)out, C, taps, residual, act, bias);
    else fz_launch(short_conv_kernel<__nv_bfloat16>, dim3(N, (C + 255) / 256), dim3(256), 0, stream, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, (const float*)state, seg, seq_row, (__nv_bfloat16*)out, C, taps, residual, act, bias);
    FZ_LAUNCH_CHECK();
    if (taps > 1 && state != nullptr && n_seg > 0)
      fz_launch(short_conv_state_kernel<__nv_bfloat16>, dim3(n_seg, (C + 255) / 256), dim3(256), 0, stream, (const __nv_bfloat16*)h, state, seg, C, taps);
  } else {
    return FZ_BAD_DTYPE;
  }
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_gated_sum(const float* a, const float* ga, const float* f, const float* gf, float* out, int N, int D,
                        int terms, float fw, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  const size_t total = (size_t)N * D;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  fz_launch(gated_sum_kernel, dim3(blocks), dim3(256), 0, stream, a, ga, f, gf, out, N, D, terms, fw);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_scale(float* x, float factor, long long total, cudaStream_t stream) {
  if (total <= 0) return FZ_OK;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  fz_launch(scale_kernel, dim3(blocks), dim3(256), 0, stream, x, factor, (size_t)total);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_select_tokens(const int* tokens, const int* src, const int* prev_ids, int* out, int N, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  fz_launch(select_tokens_kernel, dim3((N + 255) / 256), dim3(256), 0, stream, tokens, src, prev_ids, out, N);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_latent_cache_write(const float* down, const void* w, int w_dtype, float eps, const float* cos_t,
                                 const float* sin_t, int rotated, const int* pos, const int* seq_row, const int* table,
                                 int mb, void* pool, int dtype, long long page_stride, int page_size, int N, int L, int R,
                                 int max_len, int num_pages, int pairing, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (rotated < 0 || rotated > R || rotated % 2 || pairing < 0 || pairing > 1) return FZ_BAD_SHAPE;
#define FZ_LW(TW, T) do { fz_launch(latent_cache_write_kernel<TW, T>, dim3(N), dim3(128), 0, stream, down, (const TW*)w, eps, \
    cos_t, sin_t, rotated, pos, seq_row, table, mb, (T*)pool, page_stride, page_size, L, R, max_len, num_pages, err, pairing); \
    FZ_LAUNCH_CHECK(); return FZ_OK; } while (0)
  if (w_dtype == FZ_F32 && dtype == FZ_F32) FZ_LW(float, float);
  if (w_dtype == FZ_F32 && dtype == FZ_BF16) FZ_LW(float, __nv_bfloat16);
  if (w_dtype == FZ_BF16 && dtype == FZ_BF16) FZ_LW(__nv_bfloat16, __nv_bfloat16);
#undef FZ_LW
  return FZ_BAD_DTYPE;
}

FZ_API int fz_rotate_heads(const void* q, int W, int off, const float* cos_t, const float* sin_t, int rotated,
                           const int* pos, const int* seq_row, void* out, int Wo, int out_off, int dtype, int N, int H,
                           int max_len, int pairing, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (rotated < 0 || rotated > W - off || rotated % 2 || pairing < 0 || pairing > 1) return FZ_BAD_SHAPE;
  if (dtype == FZ_F32)
    fz_launch(rotate_heads_kernel<float>, dim3(N), dim3(256), 0, stream, (const float*)q, W, off, cos_t, sin_t, rotated, pos, seq_row, (float*)out, Wo, out_off, H, max_len, err, pairing);
  else if (dtype == FZ_BF16)
    fz_launch(rotate_heads_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, (const __nv_bfloat16*)q, W, off, cos_t, sin_t, rotated, pos, seq_row, (__nv_bfloat16*)out, Wo, out_off, H, max_len, err, pairing);
  else
    return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(mix_rows)
#endif
