// Row kernels of depth-averaged layers and of the hashed pair embedding, and a columnwise activation. All arithmetic is
// 32-bit; T is the dtype of a table that is read or of an activation that is written.
#include "common.cuh"
#include <math.h>
#include <stdint.h>

namespace {
// x[n] += table[r], r chosen by a hash of (previous token, token). One block per row. The block of a portion's first row
// reads the request's previous token from its state slot and then leaves the portion's last token there (no other block
// touches that slot: a request has one portion in a step).
template <typename T>
__global__ void __launch_bounds__(256)
hashed_pair_embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ seq_row,
                         const int* __restrict__ seg, int* __restrict__ state, int buckets, long long mul_prev,
                         long long mul_cur, int vocab, float* __restrict__ x, int D, int* err) {
  fz_grid_launch_dependents();
  const int n = blockIdx.x;
  const int row = seq_row[n];
  fz_grid_wait();
  if (row < 0) return;
  const int row0 = seg[4 * row], cnt = seg[4 * row + 1], pos0 = seg[4 * row + 2], slot = seg[4 * row + 3];
  const int i = n - row0;
  __shared__ int prev_s;
  if (threadIdx.x == 0) {
    int prev = 0;
    if (i > 0) prev = ids[n - 1];
    else if (slot >= 0) {
      prev = state[slot];
      state[slot] = ids[row0 + cnt - 1];
    }
    prev_s = prev;
  }
  __syncthreads();
  const int tok = ids[n], prev = prev_s;
  if (tok < 0 || tok >= vocab || prev < 0 || prev >= vocab) { if (threadIdx.x == 0) atomicOr(err, FZ_ERR_TOKEN_RANGE); return; }
  const long long r = pos0 + i == 0 ? (long long)buckets : ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
  const T* src = table + (size_t)r * D;
  float* dst = x + (size_t)n * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] += Cvt<T>::to_f(src[d]);
}

// Four neighbouring elements of sum_j coef[j] streams[j], j = 0 .. depth, plus coef[depth + 1] X: fused multiply-adds in
// rising j from zero, element by element as the scalar loops do.
__device__ __forceinline__ float4 averaged4(const float* __restrict__ st, int D, int d, int depth, const float* __restrict__ coef,
                                            float4 X) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int j = 0; j <= depth; ++j) {
    const float4 s = *(const float4*)(st + (size_t)j * D + d);
    const float c = coef[j];
    acc.x = fmaf(c, s.x, acc.x); acc.y = fmaf(c, s.y, acc.y); acc.z = fmaf(c, s.z, acc.z); acc.w = fmaf(c, s.w, acc.w);
  }
  const float c = coef[depth + 1];
  acc.x = fmaf(c, X.x, acc.x); acc.y = fmaf(c, X.y, acc.y); acc.z = fmaf(c, X.z, acc.z); acc.w = fmaf(c, X.w, acc.w);
  return acc;
}

// streams: (N, L1, D). X = x + delta; streams[n, depth + 1] = X; x = sum_j coef[j] streams[n, j], j = 0 .. depth + 1, by
// fused multiply-adds in rising j from zero. coef null (depth -1): only X is kept and x = X.
__global__ void __launch_bounds__(256)
depth_average_kernel(float* __restrict__ streams, int L1, int depth, const float* __restrict__ coef, float* __restrict__ x,
                     const float* __restrict__ delta, int D) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  float* st = streams + (size_t)n * L1 * D;
  float* xr = x + (size_t)n * D;
  const float* dr = delta != nullptr ? delta + (size_t)n * D : nullptr;
  if ((D & 3) == 0 && ((((uintptr_t)streams) | ((uintptr_t)x) | ((uintptr_t)delta)) & 15) == 0) {      // 16 bytes per access; every element's sum is the scalar loop's
    for (int d = 4 * threadIdx.x; d < D; d += 4 * blockDim.x) {
      float4 X = *(const float4*)(xr + d);
      if (dr != nullptr) { const float4 e = *(const float4*)(dr + d); X.x += e.x; X.y += e.y; X.z += e.z; X.w += e.w; }
      *(float4*)(st + (size_t)(depth + 1) * D + d) = X;
      *(float4*)(xr + d) = coef != nullptr ? averaged4(st, D, d, depth, coef, X) : X;
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float X = dr != nullptr ? xr[d] + dr[d] : xr[d];
    st[(size_t)(depth + 1) * D + d] = X;
    float acc = X;
    if (coef != nullptr) {
      acc = 0.f;
      for (int j = 0; j <= depth; ++j) acc = fmaf(coef[j], st[(size_t)j * D + d], acc);
      acc = fmaf(coef[depth + 1], X, acc);
    }
    xr[d] = acc;
  }
}

// `depth_average_kernel` and the RMS norm of its result in one pass over the row: h = w * x * rsqrt(mean(x^2) + eps) of
// the averaged x. rows == nullptr: one block per row n, the kept stream and x are written as the unfused kernel writes
// them. rows != nullptr: block r reads row rows[r] and writes only h[r] (rows[r] < 0 gives zeros). The averaged row
// waits in shared memory (D floats) between the two passes.
template <typename TH>
__global__ void __launch_bounds__(256)
depth_average_norm_kernel(float* __restrict__ streams, int L1, int depth, const float* __restrict__ coef, float* __restrict__ x,
                          const float* __restrict__ delta, int D, const float* __restrict__ w, float eps, TH* __restrict__ h,
                          const int* __restrict__ rows, int n_src, int* err) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ __align__(16) float avg[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  int n = r;
  TH* hr = h + (size_t)r * D;
  if (rows != nullptr) {
    n = rows[r];
    if (n < 0 || n >= n_src) {
      if (n >= n_src && threadIdx.x == 0) atomicOr(err, FZ_ERR_ROW_RANGE);
      for (int d = threadIdx.x; d < D; d += blockDim.x) hr[d] = Cvt<TH>::from_f(0.f);
      return;
    }
  }
  float* st = streams + (size_t)n * L1 * D;
  float* xr = x + (size_t)n * D;
  const float* dr = delta != nullptr ? delta + (size_t)n * D : nullptr;
  float ss = 0.f;
  const bool vec = (D & 3) == 0 && ((((uintptr_t)streams) | ((uintptr_t)x) | ((uintptr_t)delta)) & 15) == 0;
  for (int d = 4 * threadIdx.x; vec && d < D; d += 4 * blockDim.x) {
    float4 X = *(const float4*)(xr + d);
    if (dr != nullptr) { const float4 e = *(const float4*)(dr + d); X.x += e.x; X.y += e.y; X.z += e.z; X.w += e.w; }
    const float4 acc = averaged4(st, D, d, depth, coef, X);
    if (rows == nullptr) {
      *(float4*)(st + (size_t)(depth + 1) * D + d) = X;
      *(float4*)(xr + d) = acc;
    }
    *(float4*)(avg + d) = acc;
    ss = fmaf(acc.x, acc.x, ss); ss = fmaf(acc.y, acc.y, ss); ss = fmaf(acc.z, acc.z, ss); ss = fmaf(acc.w, acc.w, ss);
  }
  for (int d = threadIdx.x; !vec && d < D; d += blockDim.x) {
    const float X = dr != nullptr ? xr[d] + dr[d] : xr[d];
    float acc = 0.f;
    for (int j = 0; j <= depth; ++j) acc = fmaf(coef[j], st[(size_t)j * D + d], acc);
    acc = fmaf(coef[depth + 1], X, acc);
    if (rows == nullptr) {
      st[(size_t)(depth + 1) * D + d] = X;
      xr[d] = acc;
    }
    avg[d] = acc;
    ss = fmaf(acc, acc, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss * (1.0f / (float)D) + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) hr[d] = Cvt<TH>::from_f(w[d] * (avg[d] * scale));
}

// out[n, j] = act(src[n, off + j]). kind 0: tanh, 1: sigmoid, 2: silu, 3: the tanh form of gelu.
template <typename T>
__global__ void __launch_bounds__(256)
activate_kernel(const float* __restrict__ src, int ld, int off, int kind, T* __restrict__ out, int W, long long total) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / W;
    const int j = (int)(idx - n * W);
    const float z = src[n * ld + off + j];
    float v;
    if (kind == 0) v = tanhf(z);
    else if (kind == 1) v = 1.0f / (1.0f + expf(-z));
    else if (kind == 2) v = z / (1.0f + expf(-z));
    else if (kind == 3) v = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    else v = z;
    out[idx] = Cvt<T>::from_f(v);
  }
}

__device__ __forceinline__ float act_of(float z, int kind) {
  if (kind == 0) return tanhf(z);
  if (kind == 1) return 1.0f / (1.0f + expf(-z));
  if (kind == 2) return z / (1.0f + expf(-z));
  if (kind == 3) return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z;
}
__device__ __forceinline__ void st4(float* d, float4 v) { *(float4*)d = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* d, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  *(uint2*)d = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
}
__device__ __forceinline__ float4 ld4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 u = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&u.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}

// The three kernels below with four columns per thread (16-byte loads of the float32 operands), for widths, offsets and
// row pitches that are multiples of four and 16-byte aligned bases: the same values as one column per thread.
template <typename T>
__global__ void __launch_bounds__(256)
activate_vec_kernel(const float* __restrict__ src, int ld, int off, int kind, T* __restrict__ out, int W, long long quads) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int wq = W >> 2;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < quads; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / wq;
    const int j = (int)(idx - n * wq) << 2;
    const float4 z = ld4(src + n * ld + off + j);
    st4(out + n * W + j, make_float4(act_of(z.x, kind), act_of(z.y, kind), act_of(z.z, kind), act_of(z.w, kind)));
  }
}
template <typename T>
__global__ void __launch_bounds__(256)
gate_multiply_vec_kernel(const T* x, const float* __restrict__ gate, int ld, int off, int kind, T* out, int W, long long quads) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int wq = W >> 2;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < quads; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / wq;
    const int j = (int)(idx - n * wq) << 2;
    const float4 z = ld4(gate + n * ld + off + j), v = ld4(x + n * W + j);
    st4(out + n * W + j, make_float4(__fmul_rn(v.x, act_of(z.x, kind)), __fmul_rn(v.y, act_of(z.y, kind)),
                                     __fmul_rn(v.z, act_of(z.z, kind)), __fmul_rn(v.w, act_of(z.w, kind))));
  }
}
__global__ void __launch_bounds__(256)
blend_columns_vec_kernel(float* __restrict__ dst, int ldd, int doff, const float* __restrict__ src, int lds, int soff,
                         const float* __restrict__ weight, int W, long long quads) {
  fz_grid_launch_dependents();
  const float w = weight[0], keep = __fsub_rn(1.0f, w);
  fz_grid_wait();
  const int wq = W >> 2;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < quads; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / wq;
    const int j = (int)(idx - n * wq) << 2;
    float* d = dst + n * ldd + doff + j;
    const float4 a = ld4(d), b = ld4(src + n * lds + soff + j);
    st4(d, make_float4(__fadd_rn(__fmul_rn(keep, a.x), __fmul_rn(w, b.x)), __fadd_rn(__fmul_rn(keep, a.y), __fmul_rn(w, b.y)),
                       __fadd_rn(__fmul_rn(keep, a.z), __fmul_rn(w, b.z)), __fadd_rn(__fmul_rn(keep, a.w), __fmul_rn(w, b.w))));
  }
}

// out = T(x * act(gate[:, off + j])): the activation (kinds of `activate_kernel`) and the product in float32. out may be x.
template <typename T>
__global__ void __launch_bounds__(256)
gate_multiply_kernel(const T* x, const float* __restrict__ gate, int ld, int off, int kind, T* out, int W, long long total) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / W;
    const int j = (int)(idx - n * W);
    const float z = gate[n * ld + off + j];
    out[idx] = Cvt<T>::from_f(__fmul_rn(Cvt<T>::to_f(x[idx]), act_of(z, kind)));
  }
}

// dst[:, doff + j] = (1 - w) dst[:, doff + j] + w src[:, soff + j], w = weight[0]: two rounded products, then their sum.
__global__ void __launch_bounds__(256)
blend_columns_kernel(float* __restrict__ dst, int ldd, int doff, const float* __restrict__ src, int lds, int soff,
                     const float* __restrict__ weight, int W, long long total) {
  fz_grid_launch_dependents();
  const float w = weight[0], keep = __fsub_rn(1.0f, w);
  fz_grid_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / W;
    const int j = (int)(idx - n * W);
    float* d = dst + n * ldd + doff + j;
    *d = __fadd_rn(__fmul_rn(keep, *d), __fmul_rn(w, src[n * lds + soff + j]));
  }
}
}  // namespace

FZ_API int fz_hashed_pair_embed(const void* table, int dtype, const int* ids, const int* seq_row, const int* seg, int* state,
                                int buckets, long long mul_prev, long long mul_cur, int vocab, float* x, int N, int D, int* err,
                                cudaStream_t stream) {
  if (N <= 0 || D <= 0) return FZ_OK;
  if (buckets <= 0 || mul_prev < 0 || mul_cur < 0) return FZ_BAD_SHAPE;
  if (dtype == FZ_F32)
    fz_launch(hashed_pair_embed_kernel<float>, dim3(N), dim3(256), 0, stream, (const float*)table, ids, seq_row, seg, state,
              buckets, mul_prev, mul_cur, vocab, x, D, err);
  else if (dtype == FZ_BF16)
    fz_launch(hashed_pair_embed_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, seq_row,
              seg, state, buckets, mul_prev, mul_cur, vocab, x, D, err);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_depth_average(float* streams, int L1, int depth, const float* coef, float* x, const float* delta, int N, int D,
                            cudaStream_t stream) {
  if (N <= 0 || D <= 0) return FZ_OK;
  if (depth < -1 || depth + 1 >= L1 || (coef == nullptr) != (depth == -1)) return FZ_BAD_SHAPE;
  fz_launch(depth_average_kernel, dim3(N), dim3(256), 0, stream, streams, L1, depth, coef, x, delta, D);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// n_out blocks: the rows of the step (rows null, n_out = n_src) or the selected ones. w: D float32 values.
FZ_API int fz_depth_average_norm(float* streams, int L1, int depth, const float* coef, float* x, const float* delta, int n_src,
                                 int D, const float* w, float eps, void* h, int h_dtype, const int* rows, int n_out, int* err,
                                 cudaStream_t stream) {
  if (n_out <= 0 || D <= 0) return FZ_OK;
  if (depth < 0 || depth + 1 >= L1 || coef == nullptr || w == nullptr) return FZ_BAD_SHAPE;
  const size_t smem = sizeof(float) * (size_t)D;
  if (smem > 200 * 1024) return FZ_TOO_LARGE;
  if (h_dtype == FZ_F32) {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
      cudaError_t e = cudaFuncSetAttribute(depth_average_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      allowed = smem;
    }
    fz_launch(depth_average_norm_kernel<float>, dim3(n_out), dim3(256), smem, stream, streams, L1, depth, coef, x, delta, D, w,
              eps, (float*)h, rows, n_src, err);
  } else if (h_dtype == FZ_BF16) {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
      cudaError_t e = cudaFuncSetAttribute(depth_average_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      allowed = smem;
    }
    fz_launch(depth_average_norm_kernel<__nv_bfloat16>, dim3(n_out), dim3(256), smem, stream, streams, L1, depth, coef, x, delta,
              D, w, eps, (__nv_bfloat16*)h, rows, n_src, err);
  } else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_activate(const float* src, int ld, int off, int kind, void* out, int dtype, int N, int W, cudaStream_t stream) {
  const long long total = (long long)N * W;
  if (total <= 0) return FZ_OK;
  if (kind < 0 || kind > 4 || off < 0 || off + W > ld) return FZ_BAD_SHAPE;
  if (W % 4 == 0 && off % 4 == 0 && ld % 4 == 0 && (((uintptr_t)src | (uintptr_t)out) & 15) == 0 && (dtype == FZ_F32 || dtype == FZ_BF16)) {
    const long long quads = total / 4;
    long long vb = (quads + 255) / 256;
    if (vb > 148LL * 16) vb = 148LL * 16;
    if (dtype == FZ_F32) fz_launch(activate_vec_kernel<float>, dim3((int)vb), dim3(256), 0, stream, src, ld, off, kind, (float*)out, W, quads);
    else fz_launch(activate_vec_kernel<__nv_bfloat16>, dim3((int)vb), dim3(256), 0, stream, src, ld, off, kind, (__nv_bfloat16*)out, W, quads);
    FZ_LAUNCH_CHECK();
    return FZ_OK;
  }
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (dtype == FZ_F32) fz_launch(activate_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, src, ld, off, kind, (float*)out, W, total);
  else if (dtype == FZ_BF16)
    fz_launch(activate_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, src, ld, off, kind, (__nv_bfloat16*)out, W, total);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_gate_multiply(const void* x, const float* gate, int ld, int off, int kind, void* out, int dtype, int N, int W,
                            cudaStream_t stream) {
  const long long total = (long long)N * W;
  if (total <= 0) return FZ_OK;
  if (kind < 0 || kind > 4 || off < 0 || off + W > ld) return FZ_BAD_SHAPE;
  if (W % 4 == 0 && off % 4 == 0 && ld % 4 == 0 && (((uintptr_t)x | (uintptr_t)gate | (uintptr_t)out) & 15) == 0 &&
      (dtype == FZ_F32 || dtype == FZ_BF16)) {
    const long long quads = total / 4;
    long long vb = (quads + 255) / 256;
    if (vb > 148LL * 16) vb = 148LL * 16;
    if (dtype == FZ_F32)
      fz_launch(gate_multiply_vec_kernel<float>, dim3((int)vb), dim3(256), 0, stream, (const float*)x, gate, ld, off, kind, (float*)out, W, quads);
    else
      fz_launch(gate_multiply_vec_kernel<__nv_bfloat16>, dim3((int)vb), dim3(256), 0, stream, (const __nv_bfloat16*)x, gate, ld, off, kind,
                (__nv_bfloat16*)out, W, quads);
    FZ_LAUNCH_CHECK();
    return FZ_OK;
  }
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (dtype == FZ_F32)
    fz_launch(gate_multiply_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (const float*)x, gate, ld, off, kind, (float*)out, W, total);
  else if (dtype == FZ_BF16)
    fz_launch(gate_multiply_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, gate, ld, off,
              kind, (__nv_bfloat16*)out, W, total);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_blend_columns(float* dst, int ldd, int doff, const float* src, int lds, int soff, const float* weight, int N, int W,
                            cudaStream_t stream) {
  const long long total = (long long)N * W;
  if (total <= 0) return FZ_OK;
  if (doff < 0 || doff + W > ldd || soff < 0 || soff + W > lds || weight == nullptr) return FZ_BAD_SHAPE;
  if (W % 4 == 0 && doff % 4 == 0 && ldd % 4 == 0 && soff % 4 == 0 && lds % 4 == 0 && (((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const long long quads = total / 4;
    long long vb = (quads + 255) / 256;
    if (vb > 148LL * 16) vb = 148LL * 16;
    fz_launch(blend_columns_vec_kernel, dim3((int)vb), dim3(256), 0, stream, dst, ldd, doff, src, lds, soff, weight, W, quads);
    FZ_LAUNCH_CHECK();
    return FZ_OK;
  }
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  fz_launch(blend_columns_kernel, dim3((int)blocks), dim3(256), 0, stream, dst, ldd, doff, src, lds, soff, weight, W, total);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(stream_rows)
#endif
