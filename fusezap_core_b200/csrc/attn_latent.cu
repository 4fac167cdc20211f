// Attention over a paged cache of ONE vector per token that all heads share, with 32-bit arithmetic on CUDA cores: the
// float32 path of the latent attention (prompt portions and decoded tokens alike) and the general fallback of the
// bfloat16 path.
//
//   e_j: the cached vector of key j (W values); scores s_j = (q[n, h] . e_j) * scale over the keys
//   max(0, p - window + 1) <= j <= p of the row's own request (window 0: all); out[n, h] = softmax(s) . e[:, :Wv]
//   with `sink` (one float32 per head): the softmax's denominator also holds exp(sink[h]), which has no value; it
//   enters after the last chunk.
//
// One block per (token row, slice of up to 32 heads); warp w serves heads w, w + W, ... of the slice, so they share every
// load of a key. Keys are walked in chunks of 32 whose boundaries are multiples of 32 in absolute position: lane j scores
// key 32c + j, and the running (max, sum, accumulator) is updated chunk by chunk in rising c, so the order of every sum
// depends only on the row's own position and window.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int CHUNK = 32;
constexpr int MAX_WARPS = 8;
constexpr int MAX_HPW = 4;
constexpr int MAX_SLICE = MAX_WARPS * MAX_HPW;
constexpr int MAX_W = 1024, MAX_WV = 512;

template <typename T, int DPL>   // DPL: output values per lane = ceil(Wv / 32)
__global__ void attn_latent_kernel(const T* __restrict__ q, const T* __restrict__ pool, const int* __restrict__ pos,
                                   const int* __restrict__ seq_row, const int* __restrict__ table, int mb,
                                   long long page_stride, int page_size, int num_pages, T* __restrict__ out, int H, int W,
                                   int Wv, float scale, int window, int slice, int* err, const float* __restrict__ sink) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ float smem[];
  const int n = blockIdx.x, h0 = blockIdx.y * slice;      // `slice` heads per block (at most MAX_SLICE)
  const int G = min(slice, H - h0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, NW = blockDim.x >> 5;
  const int kstride = W + 1;
  float* Ks = smem;                       // [CHUNK][W + 1]
  float* Qs = Ks + CHUNK * kstride;       // [G][W]
  T* orow = out + ((size_t)n * H + h0) * Wv;
  const int row = seq_row[n];
  if (row < 0) {
    for (int i = threadIdx.x; i < G * Wv; i += blockDim.x) orow[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const int p = pos[n];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const T* qrow = q + ((size_t)n * H + h0) * W;
  for (int i = threadIdx.x; i < G * W; i += blockDim.x) Qs[i] = Cvt<T>::to_f(qrow[i]);

  float m[MAX_HPW], l[MAX_HPW], acc[MAX_HPW][DPL];
#pragma unroll
  for (int a = 0; a < MAX_HPW; ++a) {
    m[a] = -INFINITY;
    l[a] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[a][i] = 0.f;
  }
  const int* trow = table + (size_t)row * mb;
  for (int c = lo / CHUNK; c <= p / CHUNK; ++c) {
    __syncthreads();   // the previous chunk is consumed (and Qs is written, the first time)
    for (int e = threadIdx.x; e < CHUNK * W; e += blockDim.x) {
      const int j = e / W, d = e - j * W;
      const int key = c * CHUNK + j;
      float kv = 0.f;
      if (key >= lo && key <= p) {
        const int page = trow[key / page_size];
        if (page < 0 || page >= num_pages) atomicOr(err, FZ_ERR_NO_PAGE);
        else kv = Cvt<T>::to_f(pool[(long long)page * page_stride + (long long)(key % page_size) * W + d]);
      }
      Ks[j * kstride + d] = kv;
    }
    __syncthreads();
    const int key = c * CHUNK + lane;
    const bool valid = key >= lo && key <= p;
#pragma unroll
    for (int a = 0; a < MAX_HPW; ++a) {
      const int g = warp + a * NW;
      if (g >= G) break;
      const float* qh = Qs + g * W;
      const float* kr = Ks + lane * kstride;
      float s = 0.f;
      for (int d = 0; d < W; ++d) s = fmaf(qh[d], kr[d], s);
      s = valid ? s * scale : -INFINITY;
      const float mn = fmaxf(m[a], warp_max(s));       // finite: every chunk walked holds at least one visible key
      const float pj = valid ? expf(s - mn) : 0.f;
      const float corr = expf(m[a] - mn);               // 0 for the first chunk (m = -inf)
      l[a] = l[a] * corr + warp_sum(pj);
      m[a] = mn;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[a][i] *= corr;
      for (int j = 0; j < CHUNK; ++j) {
        const float pv = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          const int d = lane + 32 * i;
          if (d < Wv) acc[a][i] = fmaf(pv, Ks[j * kstride + d], acc[a][i]);
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < MAX_HPW; ++a) {
    const int g = warp + a * NW;
    if (g >= G) break;
    float corr = 1.f;
    if (sink != nullptr) {
      const float sk = sink[h0 + g], mn = fmaxf(m[a], sk);
      corr = expf(m[a] - mn);
      l[a] = l[a] * corr + expf(sk - mn);
    }
    const float inv = 1.0f / l[a];
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < Wv) orow[g * Wv + d] = Cvt<T>::from_f(acc[a][i] * corr * inv);
    }
  }
}

template <typename T, int DPL>
int launch(const void* q, const void* pool, const int* pos, const int* seq_row, const int* table, int mb,
           long long page_stride, int page_size, int num_pages, void* out, int N, int H, int W, int Wv, float scale,
           int window, const float* sink, int* err, cudaStream_t stream) {
  // heads per block: as many as share a chunk of keys in shared memory (fewer for very wide cached vectors)
  int G = H < MAX_SLICE ? H : MAX_SLICE;
  while (G > 1 && sizeof(float) * ((size_t)CHUNK * (W + 1) + (size_t)G * W) > 200 * 1024) G = (G + 1) / 2;
  const int NW = G < MAX_WARPS ? G : MAX_WARPS;
  const size_t smem = sizeof(float) * ((size_t)CHUNK * (W + 1) + (size_t)G * W);
  auto kern = attn_latent_kernel<T, DPL>;
  static size_t allowed = 48 * 1024;   // per instantiation: the attribute is raised once, outside any capture
  if (smem > allowed) {
    if (smem > 227 * 1024) return FZ_TOO_LARGE;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  fz_launch(kern, dim3(N, (H + G - 1) / G), dim3(32 * NW), smem, stream, (const T*)q, (const T*)pool, pos,
            seq_row, table, mb, page_stride, page_size, num_pages, (T*)out, H, W, Wv, scale, window, G, err, sink);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

template <typename T>
int dispatch(const void* q, const void* pool, const int* pos, const int* seq_row, const int* table, int mb,
             long long page_stride, int page_size, int num_pages, void* out, int N, int H, int W, int Wv, float scale,
             int window, const float* sink, int* err, cudaStream_t stream) {
#define FZ_GO(D) return launch<T, D>(q, pool, pos, seq_row, table, mb, page_stride, page_size, num_pages, out, N, H, W, Wv, scale, window, sink, err, stream)
  const int dpl = (Wv + 31) / 32;
  if (dpl <= 1) FZ_GO(1);
  if (dpl <= 2) FZ_GO(2);
  if (dpl <= 4) FZ_GO(4);
  if (dpl <= 8) FZ_GO(8);
  if (dpl <= 16) FZ_GO(16);
#undef FZ_GO
  return FZ_BAD_SHAPE;
}
}  // namespace

// Sizes taken: any number of heads, 0 < Wv <= W, W <= 1024, Wv <= 512.
FZ_API int fz_attn_latent_check(int H, int W, int Wv) {
  if (H <= 0 || W <= 0 || Wv <= 0 || Wv > W || W > MAX_W || Wv > MAX_WV) return FZ_BAD_SHAPE;
  if (H > 65535) return FZ_BAD_SHAPE;
  return FZ_OK;
}

FZ_API int fz_attn_latent(const void* q, const void* pool, const int* pos, const int* seq_row, const int* table, int mb,
                          long long page_stride, int page_size, int num_pages, void* out, int dtype, int N, int H, int W,
                          int Wv, float scale, int window, const float* sink, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (fz_attn_latent_check(H, W, Wv) != FZ_OK || page_size <= 0) return FZ_BAD_SHAPE;
  if (dtype == FZ_F32)
    return dispatch<float>(q, pool, pos, seq_row, table, mb, page_stride, page_size, num_pages, out, N, H, W, Wv, scale, window, sink, err, stream);
  if (dtype == FZ_BF16)
    return dispatch<__nv_bfloat16>(q, pool, pos, seq_row, table, mb, page_stride, page_size, num_pages, out, N, H, W, Wv, scale, window, sink, err, stream);
  return FZ_BAD_DTYPE;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(attn_latent)
#endif
