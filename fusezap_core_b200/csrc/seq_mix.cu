// Kernels of the recurrent mixers (retention, gated delta rule), of the windowed attention with kept first tokens and a
// sink, and of the routed experts' router and weighted sum. All arithmetic that enters a recurrence, a score, a softmax,
// a norm or a router is 32-bit; T is the activation dtype of what is read or written around them.
//
// Portions: seg[s] = (first row, rows, first position, state slot) per request of the step; a recurrent kernel walks a
// portion's tokens in order from the state in the request's slot and leaves the state there. Nothing depends on which
// other portions share the step.
#include "common.cuh"
#include <math.h>

namespace {
// ------------------------------------------------------------------------------------------ rotation + cache write
// One rotated value of a head: element i of x (dk values), turned by the angle of pair j at position p when i lies in
// the first `rotated` dimensions. pairing 0: (i, i + rotated/2); 1: (2j, 2j + 1).
__device__ __forceinline__ float rotated_value(const float* __restrict__ x, int i, int rotated, int pairing,
                                               const float* __restrict__ cs, const float* __restrict__ sn) {
  if (i >= rotated) return x[i];
  const int half = rotated >> 1;
  int j, a, b;
  if (pairing == 0) { j = i < half ? i : i - half; a = j; b = j + half; }
  else { j = i >> 1; a = 2 * j; b = a + 1; }
  float o1, o2;
  fz_rope_pair(x[a], x[b], cs[j], sn[j], o1, o2);
  return i == a ? o1 : o2;
}

// Element i of a head after its optional norm: x[i] * inv * w[i] (w null: x[i] as it is).
__device__ __forceinline__ float normed_value(const float* __restrict__ x, int i, float inv, const float* __restrict__ w) {
  return w != nullptr ? x[i] * inv * w[i] : x[i];
}
// `rotated_value` of a head that is normed first.
__device__ __forceinline__ float rotated_normed_value(const float* __restrict__ x, int i, int rotated, int pairing,
                                                      const float* __restrict__ cs, const float* __restrict__ sn, float inv,
                                                      const float* __restrict__ w) {
  if (i >= rotated) return normed_value(x, i, inv, w);
  const int half = rotated >> 1;
  int j, a, b;
  if (pairing == 0) { j = i < half ? i : i - half; a = j; b = j + half; }
  else { j = i >> 1; a = 2 * j; b = a + 1; }
  float o1, o2;
  fz_rope_pair(normed_value(x, a, inv, w), normed_value(x, b, inv, w), cs[j], sn[j], o1, o2);
  return i == a ? o1 : o2;
}

// A row of qkv is ld floats: [q heads | k heads | v heads | ...]. qn_w / kn_w (dk values, or null): every q / k head is
// divided by its root mean square (norm_eps inside the root) and multiplied by the weight before the rotation. qt_every > 0:
// q is multiplied by 1 + qt_coef * ln(floor((p + 1) / qt_every) + 1) after it.
template <typename T>
__global__ void __launch_bounds__(256)
rotate_kv_write_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       int rotated, int pairing, int max_pos, const int* __restrict__ pos, const int* __restrict__ seq_row,
                       const int* __restrict__ table, int mb, T* __restrict__ k_pool, T* __restrict__ v_pool,
                       long long page_stride, long long head_stride, long long tok_stride, int page_size, int n_pages,
                       int write, T* __restrict__ q_out, int Hq, int Hkv, int dk, int dv, const float* __restrict__ qn_w,
                       const float* __restrict__ kn_w, float norm_eps, float qt_coef, int qt_every, int* err) {
  fz_grid_launch_dependents();
  extern __shared__ __align__(16) float inv_rms[];      // [Hq + Hkv], used where a norm is asked for
  const int n = blockIdx.x;
  const int row = seq_row[n], p = pos[n];      // the step's metadata: written by the host before the step's first kernel
  fz_grid_wait();
  T* qrow = q_out + (size_t)n * Hq * dk;
  if (row < 0 || (rotated > 0 && (p < 0 || p >= max_pos))) {
    if (row >= 0) atomicOr(err, FZ_ERR_POS_RANGE);
    for (int i = threadIdx.x; i < Hq * dk; i += blockDim.x) qrow[i] = Cvt<T>::from_f(0.f);
    return;
  }
  const float* in = qkv + (size_t)n * ld;
  const int half = rotated >> 1;
  const float* cs = cos_t + (size_t)p * half;
  const float* sn = sin_t + (size_t)p * half;
  int page = -1;
  if (write) {
    page = table[(size_t)row * mb + p / page_size];
    if (page < 0 || page >= n_pages) { if (threadIdx.x == 0) atomicOr(err, FZ_ERR_NO_PAGE); page = -1; }
  }
  const int heads = write ? Hq + Hkv : Hq;
  if (qn_w != nullptr || kn_w != nullptr) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < heads; h += blockDim.x >> 5) {
      const float* x = in + (size_t)h * dk;
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) ss = fmaf(x[i], x[i], ss);
      ss = warp_sum(ss);
      if (lane == 0) inv_rms[h] = 1.0f / sqrtf(ss / (float)dk + norm_eps);
    }
    __syncthreads();
  }
  const float temp = qt_every > 0 ? 1.0f + qt_coef * logf((float)((p + 1) / qt_every) + 1.0f) : 1.0f;
  const long long at = (long long)page * page_stride + (long long)(p % page_size) * tok_stride;
  for (int e = threadIdx.x; e < heads * dk; e += blockDim.x) {
    const int head = e / dk, i = e - head * dk;
    const float* w = head < Hq ? qn_w : kn_w;
    const float v = rotated_normed_value(in + (size_t)head * dk, i, rotated, pairing, cs, sn, w != nullptr ? inv_rms[head] : 1.0f, w);
    if (head < Hq) qrow[e] = Cvt<T>::from_f(qt_every > 0 ? v * temp : v);
    else if (page >= 0) k_pool[at + (long long)(head - Hq) * head_stride + i] = Cvt<T>::from_f(v);
  }
  if (page >= 0) {
    const float* vin = in + (size_t)(Hq + Hkv) * dk;
    for (int e = threadIdx.x; e < Hkv * dv; e += blockDim.x) {
      const int head = e / dv, i = e - head * dv;
      v_pool[at + (long long)head * head_stride + i] = Cvt<T>::from_f(vin[e]);
    }
  }
}

// ------------------------------------------------------------------------------ attention: window, kept tokens, sink
// A (row, query head) pair is served by one warp. Keys are walked in chunks of 32 whose boundaries are multiples of 32 in
// absolute position, first the chunks of the kept first tokens that lie before the window, then the window's; lane j
// scores key 32c + j and the running (max, sum, accumulator) is updated chunk by chunk; the sink enters last. A chunk in
// which a pair sees no key leaves its running values exactly as they are, so the order and the bits of every sum depend
// only on the row's own position, never on the batch, the cut of the prompt, the pages used or which rows share a block.
//
// Two kernels with the same arithmetic per chunk: `sink_attention_tile_kernel` gives a block up to 32 pairs of
// consecutive rows of one portion and one kv head (the rows share every key / value load); `sink_attention_unit_kernel`
// (steps of single tokens) gives a block a run of a row's chunks and leaves (max, sum, accumulator) per run for
// `sink_attention_merge_kernel`, which adds the runs up in an order that the row's number of runs fixes.
constexpr int CHUNK = 32;
constexpr int ATT_WARPS = 8;
constexpr int MAX_PPW = 4;                         // pairs per warp
constexpr int MAX_PAIRS = ATT_WARPS * MAX_PPW;     // pairs per block

struct AttnArgs {
  const void* q; const void* k_pool; const void* v_pool;
  const int* pos; const int* seq_row; const int* seg; const int* table;
  int mb; long long page_stride, head_stride, tok_stride;
  int page_size, n_pages;
  void* out; int Hq, Hkv, dk, dv;
  float scale; int window, keep_first;
  const float* sink; int* err;
  int N;                                           // rows of the step
  int rows_per_block;                              // tile kernel: rows of a portion per block
  int unit_chunks, max_units; float* part;         // unit kernel: chunks per run, runs per row, (m, l, acc[dv]) per (row, head, run)
  float softcap;                                   // > 0: the scaled score s becomes softcap * tanh(s / softcap)
  const float* gate; int gate_ld, gate_off;        // not null: head h's result is multiplied by sigmoid(gate[n gate_ld + gate_off + h])
  int span;                                        // > 0: a row sees only the keys of its own block of `span` positions
};

// The first key a row at position p sees (kept first tokens aside): the window's start, and with a chunked mask not
// before the start of the row's own block of `span` positions. It never falls as p grows.
__device__ __forceinline__ int first_seen(int p, int window, int span) {
  int lo = window > 0 ? max(0, p - window + 1) : 0;
  if (span > 0) lo = max(lo, p - p % span);
  return lo;
}

// The chunks a row at position p walks: `first_end + 1` chunks of kept tokens, then chunks c2 .. p / CHUNK.
struct ChunkWalk {
  int lo, kept, first_end, c2, count;
  __device__ ChunkWalk(int p_first, int p_last, int window, int keep_first, int span) {
    lo = first_seen(p_first, window, span);
    kept = min(keep_first, lo);                    // keys 0 .. kept-1 are seen although they lie before the window
    first_end = kept > 0 ? (kept - 1) / CHUNK : -1;
    c2 = max(lo / CHUNK, first_end + 1);
    count = first_end + 1 + max(0, p_last / CHUNK - c2 + 1);
  }
  __device__ int chunk(int it) const { return it <= first_end ? it : c2 + (it - first_end - 1); }
};

// Sixteen bytes of T as floats.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// All threads of the block: keys and values of chunk c of kv head `kvh` that some row of the block may see, as floats.
template <typename T>
__device__ __forceinline__ void load_chunk(const AttnArgs& a, const int* trow, int kvh, int c, int lo, int kept, int p_last,
                                           float* Ks, float* Vs) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
  const T* kp = (const T*)a.k_pool;
  const T* vp = (const T*)a.v_pool;
  constexpr int VN = Vec16<T>::N;
  if (a.dk % VN == 0 && a.dv % VN == 0 && a.page_stride % VN == 0 && a.head_stride % VN == 0 && a.tok_stride % VN == 0 &&
      (reinterpret_cast<uintptr_t>(kp) & 15) == 0 && (reinterpret_cast<uintptr_t>(vp) & 15) == 0) {
    // 16 bytes per load: lane j of every warp finds the place of key 32c + j, the lanes that fetch a piece of that key
    // take it from there by a shuffle; the values stored are the same as below
    const int key = c * CHUNK + lane;
    long long off = -1;
    if (key <= p_last && (key >= lo || key < kept)) {
      const int page = trow[key / a.page_size];
      if (page < 0 || page >= a.n_pages) { if (warp == 0) atomicOr(a.err, FZ_ERR_NO_PAGE); }
      else off = (long long)page * a.page_stride + (long long)kvh * a.head_stride + (long long)(key % a.page_size) * a.tok_stride;
    }
    const int lk = a.dk / VN, lv = a.dv / VN;
    for (int base = warp * 32; base < CHUNK * lk; base += 32 * W) {
      const int e = base + lane;
      const bool in = e < CHUNK * lk;
      const int j = in ? e / lk : 0, x = e - j * lk;
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (!in) continue;
      float v[VN];
      if (oj >= 0) Vec16<T>::load(kp + oj + x * VN, v);
      else {
#pragma unroll
        for (int t = 0; t < VN; ++t) v[t] = 0.f;
      }
      float* dst = Ks + j * (a.dk + 1) + x * VN;
#pragma unroll
      for (int t = 0; t < VN; ++t) dst[t] = v[t];
    }
    for (int base = warp * 32; base < CHUNK * lv; base += 32 * W) {
      const int e = base + lane;
      const bool in = e < CHUNK * lv;
      const int j = in ? e / lv : 0, x = e - j * lv;
      const long long oj = __shfl_sync(0xffffffffu, off, j);
      if (!in) continue;
      float v[VN];
      if (oj >= 0) Vec16<T>::load(vp + oj + x * VN, v);
      else {
#pragma unroll
        for (int t = 0; t < VN; ++t) v[t] = 0.f;
      }
      float4* dst = reinterpret_cast<float4*>(Vs + j * a.dv + x * VN);
#pragma unroll
      for (int t = 0; t < VN / 4; ++t) dst[t] = make_float4(v[4 * t], v[4 * t + 1], v[4 * t + 2], v[4 * t + 3]);
    }
    return;
  }
  for (int j = warp; j < CHUNK; j += W) {
    const int key = c * CHUNK + j;
    long long off = -1;
    if (key <= p_last && (key >= lo || key < kept)) {
      const int page = trow[key / a.page_size];
      if (page < 0 || page >= a.n_pages) { if (lane == 0) atomicOr(a.err, FZ_ERR_NO_PAGE); }
      else off = (long long)page * a.page_stride + (long long)kvh * a.head_stride + (long long)(key % a.page_size) * a.tok_stride;
    }
    for (int d = lane; d < a.dk; d += 32) Ks[j * (a.dk + 1) + d] = off >= 0 ? Cvt<T>::to_f(kp[off + d]) : 0.f;
    for (int d = lane; d < a.dv; d += 32) Vs[j * a.dv + d] = off >= 0 ? Cvt<T>::to_f(vp[off + d]) : 0.f;
  }
}

// One warp, one pair, one chunk: the online-softmax update. A chunk without a visible key changes nothing.
template <int DPL>
__device__ __forceinline__ void pair_chunk(const float* qh, const float* Ks, const float* Vs, int c, int p, int lo,
                                           int keep_first, float scale, float softcap, int dk, int dv, float& m, float& l, float* acc) {
  const int lane = threadIdx.x & 31;
  const int key = c * CHUNK + lane;
  const bool valid = key <= p && (key >= lo || key < keep_first);
  const float* kr = Ks + lane * (dk + 1);
  float s = 0.f;
  for (int d = 0; d < dk; ++d) s = fmaf(qh[d], kr[d], s);
  if (softcap > 0.f) {
    s = softcap * tanhf(__fmul_rn(s, scale) / softcap);
    s = valid ? s : -INFINITY;
  } else {
    s = valid ? s * scale : -INFINITY;
  }
  const float mn = fmaxf(m, warp_max(s));
  if (mn == -INFINITY) return;                     // nothing seen so far, nothing here
  const float pj = valid ? expf(s - mn) : 0.f;
  const float corr = expf(m - mn);                 // 0 for the pair's first chunk (m = -inf), 1 where nothing is seen
  l = l * corr + warp_sum(pj);
  m = mn;
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] *= corr;
  for (int j = 0; j < CHUNK; ++j) {
    const float pv = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) acc[i] = fmaf(pv, Vs[j * dv + d], acc[i]);
    }
  }
}

// The sink (one more term of the denominator, no value), the division and the store of one pair's result.
template <typename T, int DPL>
__device__ __forceinline__ void pair_finish(const AttnArgs& a, int n, int head, float m, float l, const float* acc) {
  const int lane = threadIdx.x & 31;
  float corr = 1.f;
  if (a.sink != nullptr) {
    const float sk = a.sink[head];
    const float mn = fmaxf(m, sk);
    corr = expf(m - mn);
    l = l * corr + expf(sk - mn);
  }
  float inv = 1.0f / l;
  if (a.gate != nullptr) inv *= 1.0f / (1.0f + expf(-a.gate[(size_t)n * a.gate_ld + a.gate_off + head]));
  T* o = (T*)a.out + ((size_t)n * a.Hq + head) * a.dv;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < a.dv) o[d] = Cvt<T>::from_f(acc[i] * corr * inv);
  }
}

// grid (portions, tiles of rows_per_block rows, kv heads x slices of the group); block 32 * ATT_WARPS.
template <typename T, int DPL>   // DPL: value dims per lane = ceil(dv / 32)
__global__ void __launch_bounds__(32 * ATT_WARPS)
sink_attention_tile_kernel(const AttnArgs a) {
  fz_grid_launch_dependents();
  const int s = blockIdx.x;
  if (s == gridDim.x - 1) {                    // the block after the last portion's: rows of padding get zeros
    fz_grid_wait();
    if (blockIdx.y == 0 && blockIdx.z == 0)
      for (int n = 0; n < a.N; ++n)
        if (a.seq_row[n] < 0)
          for (int i = threadIdx.x; i < a.Hq * a.dv; i += blockDim.x) ((T*)a.out)[(size_t)n * a.Hq * a.dv + i] = Cvt<T>::from_f(0.f);
    return;
  }
  const int row0 = a.seg[4 * s], cnt = a.seg[4 * s + 1], pos0 = a.seg[4 * s + 2];
  fz_grid_wait();
  const int r0 = blockIdx.y * a.rows_per_block;
  if (r0 >= cnt) return;
  extern __shared__ __align__(16) float smem[];
  const int G_all = a.Hq / a.Hkv, slices = (G_all + MAX_PAIRS - 1) / MAX_PAIRS;
  const int kvh = blockIdx.z / slices, g_base = (blockIdx.z % slices) * MAX_PAIRS;
  const int G = min(MAX_PAIRS, G_all - g_base);
  const int nr = min(a.rows_per_block, cnt - r0);
  const int warp = threadIdx.x >> 5;
  const int dk = a.dk, dv = a.dv;
  float* Ks = smem;                            // [CHUNK][dk + 1]
  float* Vs = Ks + CHUNK * (dk + 1);           // [CHUNK][dv]
  float* Qs = Vs + CHUNK * dv;                 // [nr * G][dk]
  const int head0 = kvh * G_all + g_base;
  const T* q = (const T*)a.q;
  for (int e = threadIdx.x; e < nr * G * dk; e += blockDim.x) {
    const int pr = e / dk, d = e - pr * dk;
    Qs[e] = Cvt<T>::to_f(q[((size_t)(row0 + r0 + pr / G) * a.Hq + head0 + pr % G) * dk + d]);
  }
  float m[MAX_PPW], l[MAX_PPW], acc[MAX_PPW][DPL];
#pragma unroll
  for (int x = 0; x < MAX_PPW; ++x) {
    m[x] = -INFINITY;
    l[x] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[x][i] = 0.f;
  }
  const int p_first = pos0 + r0, p_last = p_first + nr - 1;
  const ChunkWalk walk(p_first, p_last, a.window, a.keep_first, a.span);
  const int* trow = a.table + (size_t)a.seq_row[row0] * a.mb;
  const int pairs = nr * G;
  for (int it = 0; it < walk.count; ++it) {
    const int c = walk.chunk(it);
    __syncthreads();   // the previous chunk is consumed (and Qs is written, the first time)
    load_chunk<T>(a, trow, kvh, c, walk.lo, a.keep_first, p_last, Ks, Vs);
    __syncthreads();
#pragma unroll
    for (int x = 0; x < MAX_PPW; ++x) {
      const int pr = warp + x * ATT_WARPS;
      if (pr >= pairs) break;
      const int p = p_first + pr / G;
      const int lo = first_seen(p, a.window, a.span);
      pair_chunk<DPL>(Qs + pr * dk, Ks, Vs, c, p, lo, a.keep_first, a.scale, a.softcap, dk, dv, m[x], l[x], acc[x]);
    }
  }
#pragma unroll
  for (int x = 0; x < MAX_PPW; ++x) {
    const int pr = warp + x * ATT_WARPS;
    if (pr >= pairs) break;
    pair_finish<T, DPL>(a, row0 + r0 + pr / G, head0 + pr % G, m[x], l[x], acc[x]);
  }
}

// grid (rows, kv heads x slices of the group, runs); a block walks `unit_chunks` chunks of its row and leaves, per query
// head, (m, l, acc[dv]) at part[((n Hq + head) max_units + run) (dv + 2)]. Rows of padding and runs past the row's last
// chunk leave nothing.
template <typename T, int DPL>
__global__ void __launch_bounds__(32 * ATT_WARPS)
sink_attention_unit_kernel(const AttnArgs a) {
  fz_grid_launch_dependents();
  const int n = blockIdx.x;
  const int row = a.seq_row[n], p = a.pos[n];
  fz_grid_wait();
  if (row < 0) return;
  const ChunkWalk walk(p, p, a.window, a.keep_first, a.span);
  const int it0 = blockIdx.z * a.unit_chunks;
  if (it0 >= walk.count) return;
  extern __shared__ __align__(16) float smem[];
  const int G_all = a.Hq / a.Hkv, slices = (G_all + MAX_PAIRS - 1) / MAX_PAIRS;
  const int kvh = blockIdx.y / slices, g_base = (blockIdx.y % slices) * MAX_PAIRS;
  const int G = min(MAX_PAIRS, G_all - g_base);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dk = a.dk, dv = a.dv;
  float* Ks = smem;
  float* Vs = Ks + CHUNK * (dk + 1);
  float* Qs = Vs + CHUNK * dv;                 // [G][dk]
  const int head0 = kvh * G_all + g_base;
  const T* q = (const T*)a.q + ((size_t)n * a.Hq + head0) * dk;
  for (int e = threadIdx.x; e < G * dk; e += blockDim.x) Qs[e] = Cvt<T>::to_f(q[e]);
  float m[MAX_PPW], l[MAX_PPW], acc[MAX_PPW][DPL];
#pragma unroll
  for (int x = 0; x < MAX_PPW; ++x) {
    m[x] = -INFINITY;
    l[x] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[x][i] = 0.f;
  }
  const int* trow = a.table + (size_t)row * a.mb;
  for (int it = it0; it < min(walk.count, it0 + a.unit_chunks); ++it) {
    const int c = walk.chunk(it);
    __syncthreads();
    load_chunk<T>(a, trow, kvh, c, walk.lo, a.keep_first, p, Ks, Vs);
    __syncthreads();
#pragma unroll
    for (int x = 0; x < MAX_PPW; ++x) {
      const int g = warp + x * ATT_WARPS;
      if (g >= G) break;
      pair_chunk<DPL>(Qs + g * dk, Ks, Vs, c, p, walk.lo, a.keep_first, a.scale, a.softcap, dk, dv, m[x], l[x], acc[x]);
    }
  }
#pragma unroll
  for (int x = 0; x < MAX_PPW; ++x) {
    const int g = warp + x * ATT_WARPS;
    if (g >= G) break;
    float* o = a.part + (((size_t)n * a.Hq + head0 + g) * a.max_units + blockIdx.z) * (dv + 2);
    if (lane == 0) { o[0] = m[x]; o[1] = l[x]; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) o[2 + d] = acc[x][i];
    }
  }
}

// grid (rows, query heads), MERGE_WARPS warps each: warp w adds up the runs w, w + MERGE_WARPS, ... of a row in rising
// order, warp 0 then adds the warps' sums in rising w; then the sink. The order depends on the row's number of runs only.
constexpr int MERGE_WARPS = 4;
template <typename T, int DPL>
__global__ void __launch_bounds__(32 * MERGE_WARPS)
sink_attention_merge_kernel(const AttnArgs a) {
  fz_grid_launch_dependents();
  __shared__ float sums[MERGE_WARPS][32 * DPL + 1];
  const int n = blockIdx.x, head = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = a.seq_row[n], p = a.pos[n];
  fz_grid_wait();
  const int dv = a.dv;
  if (row < 0) {
    T* o = (T*)a.out + ((size_t)n * a.Hq + head) * dv;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) o[d] = Cvt<T>::from_f(0.f);
    return;
  }
  const ChunkWalk walk(p, p, a.window, a.keep_first, a.span);
  const int runs = (walk.count + a.unit_chunks - 1) / a.unit_chunks;
  // the largest of the runs' maxima first, then every run's term with its own factor: no load waits for a sum, and the
  // order of the sums is that of the runs, whatever else the step holds
  const float* part = a.part + ((size_t)n * a.Hq + head) * a.max_units * (dv + 2);
  float m = -INFINITY;
  for (int u = lane; u < runs; u += 32) m = fmaxf(m, part[(size_t)u * (dv + 2)]);
  m = warp_max(m);
  float l = 0.f, acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int u = warp; u < runs; u += MERGE_WARPS) {
    const float* o = part + (size_t)u * (dv + 2);
    const float cb = expf(o[0] - m);               // 0 for a run that saw no key
    l = fmaf(o[1], cb, l);
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < dv) acc[i] = fmaf(o[2 + d], cb, acc[i]);
    }
  }
  if (warp > 0) {
    if (lane == 0) sums[warp][32 * DPL] = l;
#pragma unroll
    for (int i = 0; i < DPL; ++i) sums[warp][lane + 32 * i] = acc[i];
  }
  __syncthreads();
  if (warp > 0) return;
  for (int w = 1; w < MERGE_WARPS; ++w) {
    l += sums[w][32 * DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] += sums[w][lane + 32 * i];
  }
  pair_finish<T, DPL>(a, n, head, m, l, acc);
}

// ------------------------------------------------------------------------------------------------ recurrent scans
// The state of a head is a key_dim x value_dim matrix S. A thread owns DPT = 8 consecutive rows of DC = 4 neighbouring
// columns, as sixteen packed pairs: the recurrence runs on packed float32 x 2 instructions (each half rounds as the scalar
// instruction does), every key and query value read from shared memory serves four columns, and a head is spread over
// value_dim / 4 x R threads (the kernels are bound by the instructions they issue per token, not by memory). The R lanes that share the columns (R a power of two, R * 8 >= key_dim; lane = r * (32 / R)
// + group, so that neighbouring lanes read one address of shared memory) add their partial dot products with shuffles.
// State layout in memory: (slots, heads, value_dim, R * 8), so a thread's 8 values of a column are contiguous and a
// column's run is read in 32-byte pieces; rows beyond key_dim stay zero. A block covers (blockDim / R) * 4 columns of one
// head of one portion and walks the portion's tokens in chunks, staged in shared memory by all threads.
constexpr int DPT = 8;
constexpr int DC = 4;                       // value columns per thread: two packed pairs
constexpr int SCAN_MAX_THREADS = 512;
// While a chunk of tokens is computed, the inputs of the next one travel from global into a raw staging area of shared
// memory (`cp.async`, four bytes each); after the chunk they are turned into what the recurrence reads (rotated or unit
// vectors, decays, gates) in a second area. tch: tokens per chunk (16, or 8 where shared memory would not hold 16).

// Sum over the R lanes that hold the rows of one column group: they are 32 / R lanes apart.
template <int R>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = 16; o >= 32 / R; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Which column group (of the block) and which 16 rows a thread owns.
template <int R>
__device__ __forceinline__ void scan_place(int& group, int& r) {
  constexpr int per_warp = 32 / R;
  const int lane = threadIdx.x & 31;
  r = lane / per_warp;
  group = (threadIdx.x >> 5) * per_warp + lane % per_warp;
}

// The thread's 8 rows of two neighbouring columns (dkp floats apart), as pairs (column, column + 1); the second column
// is read and written only where it exists.
__device__ __forceinline__ void load_state(const float* __restrict__ p, int dkp, bool first, bool second, float2* S) {
#pragma unroll
  for (int i = 0; i < DPT; i += 4) {
    const float4 a = first ? *(const float4*)(p + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 b = second ? *(const float4*)(p + dkp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    S[i] = make_float2(a.x, b.x); S[i + 1] = make_float2(a.y, b.y); S[i + 2] = make_float2(a.z, b.z); S[i + 3] = make_float2(a.w, b.w);
  }
}
__device__ __forceinline__ void store_state(float* __restrict__ p, int dkp, bool first, bool second, const float2* S) {
#pragma unroll
  for (int i = 0; i < DPT; i += 4) {
    if (first) *(float4*)(p + i) = make_float4(S[i].x, S[i + 1].x, S[i + 2].x, S[i + 3].x);
    if (second) *(float4*)(p + dkp + i) = make_float4(S[i].y, S[i + 1].y, S[i + 2].y, S[i + 3].y);
  }
}
__device__ __forceinline__ void load8(const float* p, float* v) {       // 8 floats from shared memory, 32-byte aligned
  const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ float2 both(float v) { return make_float2(v, v); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
// Unit i of `vec` four-byte words (1 or 4) from src to dst.
__device__ __forceinline__ void cp_words(float* dst, const float* src, int i, int vec) {
  if (vec == 4) cp_async16(dst + 4 * i, src + 4 * i);
  else cp_async4(dst + i, src + i);
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Unit i of a run of values of T from global to shared: a four-byte copy in flight (T is float, or a pair of 16-bit
// values where `words` says that source, destination and length allow it), else one value copied at once.
template <typename T>
__device__ __forceinline__ void stage_unit(T* dst, const T* src, int i, bool words) {
  if (sizeof(T) == 4) cp_async4(dst + i, src + i);
  else if (words) cp_async4(dst + 2 * i, src + 2 * i);
  else dst[i] = src[i];
}

// S = decay * S + k' v^T; o = S^T q'. proj rows: [q heads | k heads | v heads | ...], ld floats apart.
template <int R>
__global__ void __launch_bounds__(SCAN_MAX_THREADS)
retention_scan_kernel(const float* __restrict__ proj, int ld, int H, int dk, int dv, int tch,
                      const float* __restrict__ decay, float key_scale, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int rotated, int pairing, int max_pos, float* __restrict__ state,
                      const int* __restrict__ seg, float* __restrict__ out, int* err) {
  fz_grid_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y;
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], pos0 = seg[4 * s + 2], slot = seg[4 * s + 3];
  fz_grid_wait();
  if (cnt <= 0 || slot < 0) return;
  if (rotated > 0 && (pos0 < 0 || pos0 + cnt > max_pos)) { if (threadIdx.x == 0) atomicOr(err, FZ_ERR_POS_RANGE); return; }
  extern __shared__ __align__(16) float smem[];
  const int NT = blockDim.x;
  const int dkp = R * DPT, COLS = NT / R * DC, half = rotated >> 1;
  float* qs = smem;                    // [tch][dkp]   what the recurrence reads
  float* ks = qs + tch * dkp;          // [tch][dkp]
  float* vs = ks + tch * dkp;          // [tch][COLS]
  float* rq = vs + tch * COLS;         // [tch][dk]    raw: as the projections left them
  float* rk = rq + tch * dk;           // [tch][dk]
  float* rv = rk + tch * dk;           // [tch][COLS]
  float* rc = rv + tch * COLS;         // [tch][half]  the rows of the cosine and sine tables
  float* rs = rc + tch * half;         // [tch][half]
  int group, r;
  scan_place<R>(group, r);
  const int col0 = blockIdx.z * COLS, col = col0 + group * DC;      // this thread's first column
  const int ncols = min(COLS, dv - col0);
  float* sp = state + (((size_t)slot * H + h) * dv + col) * dkp + r * DPT;
  const bool has[DC] = {col < dv, col + 1 < dv, col + 2 < dv, col + 3 < dv};
  float2 S[DC / 2][DPT];
  load_state(sp, dkp, has[0], has[1], S[0]);
  load_state(sp + 2 * (size_t)dkp, dkp, has[2], has[3], S[1]);
  const float2 dec = both(decay[h]);
  // what a token brings: q, k, its columns of v, cosines, sines; in copies of 16 bytes where every run starts on a 16-byte
  // boundary and has a length that is a multiple of four, else of 4 bytes
  const int vec = ((dk | ld | dv | ncols | half) & 3) == 0 && aligned16(proj) && (half == 0 || (aligned16(cos_t) && aligned16(sin_t))) ? 4 : 1;
  const int uq = dk / vec, uv = ncols / vec, uh = half / vec;
  const int per_token = 2 * uq + uv + 2 * uh;
  auto issue = [&](int t0) {
    const int tc = min(tch, cnt - t0);
    for (int e = threadIdx.x; e < tc * per_token; e += NT) {
      const int tt = e / per_token;
      int i = e - tt * per_token;
      const float* in = proj + (size_t)(row0 + t0 + tt) * ld;
      if (i < uq) { cp_words(rq + tt * dk, in + (size_t)h * dk, i, vec); continue; }
      i -= uq;
      if (i < uq) { cp_words(rk + tt * dk, in + (size_t)(H + h) * dk, i, vec); continue; }
      i -= uq;
      if (i < uv) { cp_words(rv + tt * COLS, in + (size_t)2 * H * dk + (size_t)h * dv + col0, i, vec); continue; }
      i -= uv;
      if (i < uh) cp_words(rc + tt * half, cos_t + (size_t)(pos0 + t0 + tt) * half, i, vec);
      else cp_words(rs + tt * half, sin_t + (size_t)(pos0 + t0 + tt) * half, i - uh, vec);
    }
    cp_async_commit();
  };
  auto cook = [&](int t0) {
    const int tc = min(tch, cnt - t0);
    for (int e = threadIdx.x; e < tc * dkp; e += NT) {
      const int tt = e / dkp, i = e - tt * dkp;
      float qv = 0.f, kv = 0.f;
      if (i < dk) {
        qv = rotated_value(rq + tt * dk, i, rotated, pairing, rc + tt * half, rs + tt * half);
        kv = __fmul_rn(rotated_value(rk + tt * dk, i, rotated, pairing, rc + tt * half, rs + tt * half), key_scale);
      }
      qs[e] = qv;
      ks[e] = kv;
    }
    for (int e = threadIdx.x; e < tc * COLS; e += NT) {
      const int c = e % COLS;
      vs[e] = c < ncols ? rv[e] : 0.f;
    }
  };

  issue(0);
  cp_async_wait();
  __syncthreads();
  cook(0);
  __syncthreads();
  for (int t0 = 0; t0 < cnt; t0 += tch) {
    const int tc = min(tch, cnt - t0);
    const bool more = t0 + tch < cnt;
    if (more) issue(t0 + tch);
    float* dst = out + (size_t)(row0 + t0) * H * dv + (size_t)h * dv + col;
#pragma unroll 2
    for (int tt = 0; tt < tc; ++tt, dst += (size_t)H * dv) {
      const float4 v4 = *(const float4*)(vs + tt * COLS + group * DC);
      const float2 v[DC / 2] = {make_float2(v4.x, v4.y), make_float2(v4.z, v4.w)};
      float kk[DPT], qq[DPT];
      load8(ks + tt * dkp + r * DPT, kk);
      load8(qs + tt * dkp + r * DPT, qq);
      float2 o[DC / 2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const float2 k2 = both(kk[i]), q2 = both(qq[i]);
#pragma unroll
        for (int j = 0; j < DC / 2; ++j) {
          S[j][i] = __ffma2_rn(dec, S[j][i], __fmul2_rn(k2, v[j]));
          o[j] = __ffma2_rn(S[j][i], q2, o[j]);
        }
      }
      const float res[DC] = {lanes_sum<R>(o[0].x), lanes_sum<R>(o[0].y), lanes_sum<R>(o[1].x), lanes_sum<R>(o[1].y)};
      if (r == 0) {
#pragma unroll
        for (int j = 0; j < DC; ++j)
          if (has[j]) dst[j] = res[j];
      }
    }
    if (more) {
      cp_async_wait();
      __syncthreads();               // the next chunk's raw inputs have arrived; every thread is done with this chunk
      cook(t0 + tch);
      __syncthreads();
    }
  }
  store_state(sp, dkp, has[0], has[1], S[0]);
  store_state(sp + 2 * (size_t)dkp, dkp, has[2], has[3], S[1]);
}

// S = g * S (rows); u = beta (v - S^T k^); S += k^ u^T; o = S^T q^. qkv rows: [q (Hk dk) | k (Hk dk) | v (H dv)] of T.
template <typename T, int R>
__global__ void __launch_bounds__(SCAN_MAX_THREADS)
gated_delta_scan_kernel(const T* __restrict__ qkv, int H, int Hk, int dk, int dv, int tch,
                        const float* __restrict__ high, int ldh, const float* __restrict__ beta,
                        const float* __restrict__ a_log, const float* __restrict__ dt_bias, float unit_eps, float q_scale,
                        float* __restrict__ state, const int* __restrict__ seg, float* __restrict__ out) {
  fz_grid_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y;
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], slot = seg[4 * s + 3];
  fz_grid_wait();
  if (cnt <= 0 || slot < 0) return;
  extern __shared__ __align__(16) float smem[];
  const int NT = blockDim.x;
  const int dkp = R * DPT, COLS = NT / R * DC;
  const int dke = (dk + 1) & ~1, cole = (COLS + 1) & ~1;      // raw rows of T start on four-byte boundaries
  float* qs = smem;                    // [tch][dkp]   what the recurrence reads
  float* ks = qs + tch * dkp;
  float* gs = ks + tch * dkp;
  float* vs = gs + tch * dkp;          // [tch][COLS]
  float* bs = vs + tch * COLS;         // [tch]
  float* ra = bs + tch;                // [tch][dk]    raw: decay inputs
  float* rb = ra + tch * dk;           // [tch]        raw: beta before the sigmoid
  T* rq = (T*)(rb + tch);              // [tch][dke]   raw: q, k, v after the convolution
  T* rk = rq + tch * dke;
  T* rv = rk + tch * dke;              // [tch][cole]
  int group, r;
  scan_place<R>(group, r);
  const int col0 = blockIdx.z * COLS, col = col0 + group * DC;      // this thread's first column
  const int ncols = min(COLS, dv - col0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kh = h / (H / Hk);
  const int C = 2 * Hk * dk + H * dv;
  // 16-bit values travel in pairs where every run starts on a four-byte boundary and has an even length
  const bool words = sizeof(T) == 4 || (((dk | dv | C | col0 | ncols) & 1) == 0 && ((uintptr_t)qkv & 3) == 0);
  float* sp = state + (((size_t)slot * H + h) * dv + col) * dkp + r * DPT;
  const bool has[DC] = {col < dv, col + 1 < dv, col + 2 < dv, col + 3 < dv};
  float2 S[DC / 2][DPT];
  load_state(sp, dkp, has[0], has[1], S[0]);
  load_state(sp + 2 * (size_t)dkp, dkp, has[2], has[3], S[1]);
  const float rate = expf(a_log[h]);
  const bool pairs = sizeof(T) == 2 && words;
  const int uq = pairs ? dk / 2 : dk, uv = pairs ? ncols / 2 : ncols;      // copies per run of q or k, and of v
  const int avec = ((dk | ldh) & 3) == 0 && aligned16(high) ? 4 : 1;      // the float32 decay inputs: 16 bytes a copy where aligned
  const int ua = dk / avec;
  const int per_token = 2 * uq + uv + ua + 1;
  auto issue = [&](int t0) {
    const int tc = min(tch, cnt - t0);
    for (int e = threadIdx.x; e < tc * per_token; e += NT) {
      const int tt = e / per_token;
      int i = e - tt * per_token;
      const size_t n = (size_t)(row0 + t0 + tt);
      const T* in = qkv + n * C;
      if (i < uq) { stage_unit(rq + tt * dke, in + (size_t)kh * dk, i, words); continue; }
      i -= uq;
      if (i < uq) { stage_unit(rk + tt * dke, in + (size_t)(Hk + kh) * dk, i, words); continue; }
      i -= uq;
      if (i < uv) { stage_unit(rv + tt * cole, in + (size_t)2 * Hk * dk + (size_t)h * dv + col0, i, words); continue; }
      i -= uv;
      if (i < ua) cp_words(ra + tt * dk, high + n * ldh + (size_t)h * dk, i, avec);
      else cp_async4(rb + tt, beta + n * H + h);
    }
    cp_async_commit();
  };
  auto cook = [&](int t0) {
    const int tc = min(tch, cnt - t0);
    for (int tt = warp; tt < tc; tt += NT / 32) {      // a warp cooks a token: unit vectors, decays, beta
      const T* qin = rq + tt * dke;
      const T* kin = rk + tt * dke;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float a = Cvt<T>::to_f(qin[i]), b = Cvt<T>::to_f(kin[i]);
        sq = fmaf(a, a, sq);
        sk = fmaf(b, b, sk);
      }
      const float nq = sqrtf(warp_sum(sq) + unit_eps), nk = sqrtf(warp_sum(sk) + unit_eps);
      for (int i = lane; i < dkp; i += 32) {
        float qv = 0.f, kv = 0.f, gv = 0.f;
        if (i < dk) {
          qv = __fmul_rn(__fdiv_rn(Cvt<T>::to_f(qin[i]), nq), q_scale);
          kv = __fdiv_rn(Cvt<T>::to_f(kin[i]), nk);
          const float a = ra[tt * dk + i] + dt_bias[(size_t)h * dk + i];
          const float soft = a > 20.f ? a : log1pf(expf(a));
          gv = expf(-rate * soft);
        }
        qs[tt * dkp + i] = qv;
        ks[tt * dkp + i] = kv;
        gs[tt * dkp + i] = gv;
      }
      if (lane == 0) bs[tt] = 1.0f / (1.0f + expf(-rb[tt]));
    }
    for (int e = threadIdx.x; e < tc * COLS; e += NT) {
      const int tt = e / COLS, c = e - tt * COLS;
      vs[e] = c < ncols ? Cvt<T>::to_f(rv[tt * cole + c]) : 0.f;
    }
  };

  issue(0);
  cp_async_wait();
  __syncthreads();
  cook(0);
  __syncthreads();
  for (int t0 = 0; t0 < cnt; t0 += tch) {
    const int tc = min(tch, cnt - t0);
    const bool more = t0 + tch < cnt;
    if (more) issue(t0 + tch);
    float* dst = out + (size_t)(row0 + t0) * H * dv + (size_t)h * dv + col;
#pragma unroll 2
    for (int tt = 0; tt < tc; ++tt, dst += (size_t)H * dv) {
      const float4 v4 = *(const float4*)(vs + tt * COLS + group * DC);
      const float b = bs[tt];
      float kk[DPT], qq[DPT], gg[DPT];
      load8(ks + tt * dkp + r * DPT, kk);
      load8(qs + tt * dkp + r * DPT, qq);
      load8(gs + tt * dkp + r * DPT, gg);
      float2 ksum[DC / 2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const float2 g2 = both(gg[i]), k2 = both(kk[i]);
#pragma unroll
        for (int j = 0; j < DC / 2; ++j) {
          S[j][i] = __fmul2_rn(g2, S[j][i]);
          ksum[j] = __ffma2_rn(S[j][i], k2, ksum[j]);
        }
      }
      const float2 u[DC / 2] = {make_float2(__fmul_rn(b, v4.x - lanes_sum<R>(ksum[0].x)), __fmul_rn(b, v4.y - lanes_sum<R>(ksum[0].y))),
                                make_float2(__fmul_rn(b, v4.z - lanes_sum<R>(ksum[1].x)), __fmul_rn(b, v4.w - lanes_sum<R>(ksum[1].y)))};
      float2 o[DC / 2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const float2 k2 = both(kk[i]), q2 = both(qq[i]);
#pragma unroll
        for (int j = 0; j < DC / 2; ++j) {
          S[j][i] = __ffma2_rn(k2, u[j], S[j][i]);
          o[j] = __ffma2_rn(S[j][i], q2, o[j]);
        }
      }
      const float res[DC] = {lanes_sum<R>(o[0].x), lanes_sum<R>(o[0].y), lanes_sum<R>(o[1].x), lanes_sum<R>(o[1].y)};
      if (r == 0) {
#pragma unroll
        for (int j = 0; j < DC; ++j)
          if (has[j]) dst[j] = res[j];
      }
    }
    if (more) {
      cp_async_wait();
      __syncthreads();
      cook(t0 + tch);
      __syncthreads();
    }
  }
  store_state(sp, dkp, has[0], has[1], S[0]);
  store_state(sp + 2 * (size_t)dkp, dkp, has[2], has[3], S[1]);
}

// S = diag(d) S - (a u)(u^T S) + k v^T, both products from the state before the token; o = S^T r. proj rows (ld floats):
// [r (H dk) | k (H dk) | v (H dv) | ...], the removal inputs (H dk) from column off_a on; din (N, H dk): the decay inputs.
// u = k / sqrt(sum k^2 + unit_eps), d = exp(-rate * sigmoid(din + dbias)), a = sigmoid(ain + abias), per key channel.
template <int R>
__global__ void __launch_bounds__(SCAN_MAX_THREADS)
general_delta_scan_kernel(const float* __restrict__ proj, int ld, int H, int dk, int dv, int off_a, int tch,
                          const float* __restrict__ din, const float* __restrict__ dbias, const float* __restrict__ abias,
                          float rate, float unit_eps, float* __restrict__ state, const int* __restrict__ seg,
                          float* __restrict__ out) {
  fz_grid_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y;
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], slot = seg[4 * s + 3];
  fz_grid_wait();
  if (cnt <= 0 || slot < 0) return;
  extern __shared__ __align__(16) float smem[];
  const int NT = blockDim.x;
  const int dkp = R * DPT, COLS = NT / R * DC;
  float* rs = smem;                    // [tch][dkp]   what the recurrence reads: r
  float* ks = rs + tch * dkp;          //              k
  float* us = ks + tch * dkp;          //              the unit key
  float* ds = us + tch * dkp;          //              the decay
  float* ns = ds + tch * dkp;          //              -(a * u)
  float* vs = ns + tch * dkp;          // [tch][COLS]
  float* rr = vs + tch * COLS;         // [tch][dk]    raw: as the projections left them
  float* rk = rr + tch * dk;
  float* ra = rk + tch * dk;           //              removal inputs
  float* rd = ra + tch * dk;           //              decay inputs
  float* rv = rd + tch * dk;           // [tch][COLS]
  int group, r;
  scan_place<R>(group, r);
  const int col0 = blockIdx.z * COLS, col = col0 + group * DC;      // this thread's first column
  const int ncols = min(COLS, dv - col0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* sp = state + (((size_t)slot * H + h) * dv + col) * dkp + r * DPT;
  const bool has[DC] = {col < dv, col + 1 < dv, col + 2 < dv, col + 3 < dv};
  float2 S[DC / 2][DPT];
  load_state(sp, dkp, has[0], has[1], S[0]);
  load_state(sp + 2 * (size_t)dkp, dkp, has[2], has[3], S[1]);
  // copies of 16 bytes where every run starts on a 16-byte boundary and has a length that is a multiple of four
  const int vec = ((dk | ld | dv | ncols | off_a | (H * dk)) & 3) == 0 && aligned16(proj) && aligned16(din) ? 4 : 1;
  const int uq = dk / vec, uv = ncols / vec;
  const int per_token = 4 * uq + uv;
  auto issue = [&](int t0) {
    const int tc = min(tch, cnt - t0);
    for (int e = threadIdx.x; e < tc * per_token; e += NT) {
      const int tt = e / per_token;
      int i = e - tt * per_token;
      const size_t n = (size_t)(row0 + t0 + tt);
      const float* in = proj + n * ld;
      if (i < uq) { cp_words(rr + tt * dk, in + (size_t)h * dk, i, vec); continue; }
      i -= uq;
      if (i < uq) { cp_words(rk + tt * dk, in + (size_t)(H + h) * dk, i, vec); continue; }
      i -= uq;
      if (i < uq) { cp_words(ra + tt * dk, in + off_a + (size_t)h * dk, i, vec); continue; }
      i -= uq;
      if (i < uq) { cp_words(rd + tt * dk, din + n * H * dk + (size_t)h * dk, i, vec); continue; }
      i -= uq;
      cp_words(rv + tt * COLS, in + (size_t)2 * H * dk + (size_t)h * dv + col0, i, vec);
    }
    cp_async_commit();
  };
  auto cook = [&](int t0) {
    const int tc = min(tch, cnt - t0);
    for (int tt = warp; tt < tc; tt += NT / 32) {      // a warp cooks a token: the unit key, the decay, the removal rate
      const float* kin = rk + tt * dk;
      float sk = 0.f;
      for (int i = lane; i < dk; i += 32) sk = fmaf(kin[i], kin[i], sk);
      const float nk = sqrtf(warp_sum(sk) + unit_eps);
      for (int i = lane; i < dkp; i += 32) {
        float rv_ = 0.f, kv = 0.f, uv_ = 0.f, dv_ = 0.f, nv = 0.f;
        if (i < dk) {
          rv_ = rr[tt * dk + i];
          kv = kin[i];
          uv_ = __fdiv_rn(kv, nk);
          const float zd = rd[tt * dk + i] + dbias[(size_t)h * dk + i];
          dv_ = expf(-rate * (1.0f / (1.0f + expf(-zd))));
          const float za = ra[tt * dk + i] + abias[(size_t)h * dk + i];
          nv = -(uv_ * (1.0f / (1.0f + expf(-za))));
        }
        rs[tt * dkp + i] = rv_;
        ks[tt * dkp + i] = kv;
        us[tt * dkp + i] = uv_;
        ds[tt * dkp + i] = dv_;
        ns[tt * dkp + i] = nv;
      }
    }
    for (int e = threadIdx.x; e < tc * COLS; e += NT) {
      const int c = e % COLS;
      vs[e] = c < ncols ? rv[e] : 0.f;
    }
  };

  issue(0);
  cp_async_wait();
  __syncthreads();
  cook(0);
  __syncthreads();
  for (int t0 = 0; t0 < cnt; t0 += tch) {
    const int tc = min(tch, cnt - t0);
    const bool more = t0 + tch < cnt;
    if (more) issue(t0 + tch);
    float* dst = out + (size_t)(row0 + t0) * H * dv + (size_t)h * dv + col;
#pragma unroll 2
    for (int tt = 0; tt < tc; ++tt, dst += (size_t)H * dv) {
      const float4 v4 = *(const float4*)(vs + tt * COLS + group * DC);
      const float2 v[DC / 2] = {make_float2(v4.x, v4.y), make_float2(v4.z, v4.w)};
      float kk[DPT], qq[DPT], uu[DPT], dd[DPT], nn[DPT];
      load8(us + tt * dkp + r * DPT, uu);
      float2 back[DC / 2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const float2 u2 = both(uu[i]);
#pragma unroll
        for (int j = 0; j < DC / 2; ++j) back[j] = __ffma2_rn(S[j][i], u2, back[j]);
      }
      const float2 b[DC / 2] = {make_float2(lanes_sum<R>(back[0].x), lanes_sum<R>(back[0].y)),
                                make_float2(lanes_sum<R>(back[1].x), lanes_sum<R>(back[1].y))};
      load8(ks + tt * dkp + r * DPT, kk);
      load8(rs + tt * dkp + r * DPT, qq);
      load8(ds + tt * dkp + r * DPT, dd);
      load8(ns + tt * dkp + r * DPT, nn);
      float2 o[DC / 2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        const float2 k2 = both(kk[i]), q2 = both(qq[i]), d2 = both(dd[i]), n2 = both(nn[i]);
#pragma unroll
        for (int j = 0; j < DC / 2; ++j) {
          S[j][i] = __ffma2_rn(d2, S[j][i], __ffma2_rn(k2, v[j], __fmul2_rn(n2, b[j])));
          o[j] = __ffma2_rn(S[j][i], q2, o[j]);
        }
      }
      const float res[DC] = {lanes_sum<R>(o[0].x), lanes_sum<R>(o[0].y), lanes_sum<R>(o[1].x), lanes_sum<R>(o[1].y)};
      if (r == 0) {
#pragma unroll
        for (int j = 0; j < DC; ++j)
          if (has[j]) dst[j] = res[j];
      }
    }
    if (more) {
      cp_async_wait();
      __syncthreads();
      cook(t0 + tch);
      __syncthreads();
    }
  }
  store_state(sp, dkp, has[0], has[1], S[0]);
  store_state(sp + 2 * (size_t)dkp, dkp, has[2], has[3], S[1]);
}

// out[n, h, c] = o / sqrt(mean_c o^2 + eps) * w[c] * act(gate[n, goff + h dv + c]); a warp per (row, head).
template <typename TO>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, int H, int dv, const float* __restrict__ w, int w_per_head, float eps,
                      const float* __restrict__ gate, int ldg, int goff, int act, const int* __restrict__ seq_row,
                      TO* __restrict__ out) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
  const bool pad = seq_row[n] < 0;
  for (int h = warp; h < H; h += W) {
    const float* x = o + ((size_t)n * H + h) * dv;
    TO* y = out + ((size_t)n * H + h) * dv;
    if (pad) {
      for (int c = lane; c < dv; c += 32) y[c] = Cvt<TO>::from_f(0.f);
      continue;
    }
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(x[c], x[c], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
      float v = x[c] * inv;
      if (w != nullptr) v *= w[w_per_head ? h * dv + c : c];
      if (gate != nullptr) {
        const float z = gate[(size_t)n * ldg + goff + (size_t)h * dv + c];
        const float sg = 1.0f / (1.0f + expf(-z));
        v *= act == 2 ? z * sg : sg;
      }
      y[c] = Cvt<TO>::from_f(v);
    }
  }
}

// ------------------------------------------------------------------------------------------------ router
// A warp per row: softmax over the E router logits, then lane 0 picks the groups and the experts. Scores of chosen
// experts are overwritten with -1 in shared memory (scores are never negative), so each is picked once.
constexpr int ROUTER_WARPS = 4;
__global__ void __launch_bounds__(32 * ROUTER_WARPS)
router_topk_kernel(const float* __restrict__ logits, int ld, int N, int E, int top, int groups, int keep, int renorm,
                   const int* __restrict__ seq_row, int* __restrict__ choice, float* __restrict__ weight) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * ROUTER_WARPS + warp;
  if (n >= N) return;
  float* s = smem + (size_t)warp * (E + groups + top);
  float* gmax = s + E;
  float* picked = gmax + groups;                       // the chosen scores, until their sum is known
  if (seq_row[n] < 0) {
    for (int k = lane; k < top; k += 32) { choice[(size_t)n * top + k] = 0; weight[(size_t)n * top + k] = 0.f; }
    return;
  }
  const float* z = logits + (size_t)n * ld;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float v = expf(z[e] - mx); s[e] = v; sum += v; }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) s[e] = __fdiv_rn(s[e], sum);
  __syncwarp();
  const int per = E / groups;
  for (int g = lane; g < groups; g += 32) {
    float v = -1.f;
    for (int e = g * per; e < (g + 1) * per; ++e) v = fmaxf(v, s[e]);
    gmax[g] = v;
  }
  __syncwarp();
  if (lane == 0) {
    // the groups that are not kept lose their experts: groups - keep times, strike the worst group (the higher index
    // among equals, so that the lower index stays)
    for (int d = 0; d < groups - keep; ++d) {
      int worst = -1;
      float wv = 0.f;
      for (int g = 0; g < groups; ++g) {
        if (gmax[g] < -1.5f) continue;                 // already struck
        if (worst < 0 || !(gmax[g] > wv)) { worst = g; wv = gmax[g]; }
      }
      gmax[worst] = -2.f;
      for (int e = worst * per; e < (worst + 1) * per; ++e) s[e] = -1.f;
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < E; ++e)
        if (s[e] > bv) { best = e; bv = s[e]; }
      if (best < 0) {                                  // scores that are not numbers: any expert not yet taken
        for (int e = 0; e < E && best < 0; ++e)
          if (!(s[e] == -1.f)) best = e;
        if (best < 0) best = 0;
        bv = 0.f;
      }
      choice[(size_t)n * top + k] = best;
      picked[k] = bv;
      total += bv;
      s[best] = -1.f;
    }
    for (int k = 0; k < top; ++k) weight[(size_t)n * top + k] = renorm ? __fdiv_rn(picked[k], total) : picked[k];
  }
}

// out[n] = scale * (add[n] + sum_k w[n, k] terms[n top + k] (+ sigmoid(gl[n, col]) shared[n])); a null gl counts as a gate
// of 1, a null add as zero, and the product with scale is left out when it is 1; rows of padding give zeros.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ terms, const float* __restrict__ w, int top, const float* __restrict__ shared,
                   const float* __restrict__ gl, int ldg, int col, const int* __restrict__ seq_row, float* __restrict__ out,
                   int N, int D, const float* __restrict__ add, float scale) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  const bool pad = seq_row[n] < 0;
  float sg = 1.f;
  if (!pad && shared != nullptr && gl != nullptr) sg = 1.0f / (1.0f + expf(-gl[(size_t)n * ldg + col]));
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
    float acc = 0.f;
    if (!pad) {
      for (int k = 0; k < top; ++k) acc = __fmaf_rn(w[(size_t)n * top + k], terms[((size_t)n * top + k) * D + d], acc);
      if (shared != nullptr) acc = __fmaf_rn(sg, shared[(size_t)n * D + d], acc);
      if (add != nullptr) acc = __fadd_rn(acc, add[(size_t)n * D + d]);
      if (scale != 1.f) acc = __fmul_rn(acc, scale);
    }
    out[(size_t)n * D + d] = acc;
  }
}

// ------------------------------------------------------------------------------ real-gated linear recurrent unit
// Per channel c of part b (W / B channels each): r = sigmoid(g_r + bias), i = sigmoid(g_i + bias),
// a = exp(-k_c r) with k_c = sharpness * softplus(lam_c), S <- a S + sqrt(1 - a^2) (i u), out = S y. Everything in
// float32 with explicit roundings, so that the two forms below give the same bits: 1 - a^2 is taken as -expm1(-2 k_c r),
// which keeps its digits where a is close to one.
//
// Long portions run in two launches: `rglru_cook_kernel` (every (row, channel) on its own) overwrites the two gate
// inputs by a and b = sqrt(1 - a^2) i u, and the scan, a thread per (portion, channel), walks the portion's tokens with
// one fused multiply-add each, sixteen tokens' loads in flight. What bounds it is how many loads the SMs in use keep in
// flight, so a long portion's channels are spread over as many SMs as there are half warps of channels. Steps of short portions (decoded tokens) run the scan
// alone, which then cooks a and b itself.
__device__ __forceinline__ float rglru_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ void rglru_cook(float gr, float gi, float br, float bi, float k, float u, float& a, float& b) {
  const float r = 1.0f / (1.0f + expf(-__fadd_rn(gr, br)));
  const float i = 1.0f / (1.0f + expf(-__fadd_rn(gi, bi)));
  const float la = -__fmul_rn(k, r);
  a = expf(la);
  b = __fmul_rn(sqrtf(-expm1f(__fmul_rn(2.f, la))), __fmul_rn(i, u));
}

template <typename T>
__global__ void __launch_bounds__(256)
rglru_cook_kernel(const T* __restrict__ u, float* __restrict__ gates, const float* __restrict__ gbias,
                  const float* __restrict__ lam, float sharp, const int* __restrict__ seq_row, int W, int bw, long long total) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / W;
    const int c = (int)(idx - n * W);
    if (seq_row[n] < 0) continue;
    const int part = c / bw, gcol = part * 2 * bw + (c - part * bw);
    float* g = gates + n * 2 * W + gcol;
    float a, b;
    rglru_cook(g[0], g[bw], gbias[gcol], gbias[gcol + bw], __fmul_rn(sharp, rglru_softplus(lam[c])), Cvt<T>::to_f(u[idx]), a, b);
    g[0] = a;
    g[bw] = b;
  }
}

template <typename T, bool COOKED>
__global__ void __launch_bounds__(64)
rglru_scan_kernel(const T* __restrict__ u, const float* __restrict__ gates, const float* __restrict__ gbias,
                  const float* __restrict__ lam, const T* __restrict__ y, float sharp, float* __restrict__ state,
                  const int* __restrict__ seg, T* __restrict__ out, int W, int bw) {
  fz_grid_launch_dependents();
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], slot = seg[4 * s + 3];
  int gcol = 0;
  float k = 0.f, br = 0.f, bi = 0.f;
  if (c < W) {
    const int part = c / bw;
    gcol = part * 2 * bw + (c - part * bw);
    if (!COOKED) {
      k = __fmul_rn(sharp, rglru_softplus(lam[c]));
      br = gbias[gcol];
      bi = gbias[gcol + bw];
    }
  }
  fz_grid_wait();
  if (c >= W || cnt <= 0 || slot < 0) return;
  float S = state[(size_t)slot * W + c];
  constexpr int RGLRU_AHEAD = 16;      // tokens whose loads are in flight at once
  for (int t0 = 0; t0 < cnt; t0 += RGLRU_AHEAD) {
    float a[RGLRU_AHEAD], b[RGLRU_AHEAD], yy[RGLRU_AHEAD];
#pragma unroll
    for (int i = 0; i < RGLRU_AHEAD; ++i) {
      a[i] = 1.f; b[i] = 0.f; yy[i] = 0.f;
      if (t0 + i < cnt) {
        const size_t n = (size_t)(row0 + t0 + i);
        const float* g = gates + n * 2 * W + gcol;
        yy[i] = Cvt<T>::to_f(y[n * W + c]);
        if (COOKED) { a[i] = g[0]; b[i] = g[bw]; }
        else rglru_cook(g[0], g[bw], br, bi, k, Cvt<T>::to_f(u[n * W + c]), a[i], b[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < RGLRU_AHEAD; ++i) {
      if (t0 + i < cnt) {
        S = __fmaf_rn(a[i], S, b[i]);
        out[(size_t)(row0 + t0 + i) * W + c] = Cvt<T>::from_f(__fmul_rn(S, yy[i]));
      }
    }
  }
  state[(size_t)slot * W + c] = S;
}

// The scan of long portions where the channels pair up (W and W / B even): a thread owns two neighbouring channels, and
// the coefficients and gate values of the next 32 or 48 tokens travel into the thread's own places in a ring of stages
// in shared memory (`cp.async`, 8 and 4 bytes) while the sixteen in hand are walked, so a thread waits for memory once
// per portion, not once per sixteen tokens. A thread reads only what it copied itself: `cp.async.wait_group` orders that, no barrier
// is needed. Same arithmetic and bits as `rglru_scan_kernel<T, true>`.
template <typename T> struct PairOf;
template <> struct PairOf<float> { using type = float2; static __device__ __forceinline__ float2 f(float2 v) { return v; } };
template <> struct PairOf<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ float2 f(__nv_bfloat162 v) { return __bfloat1622float2(v); }
};
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src) : "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait_n() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void store_pair(float* p, float x, float y) { *(float2*)p = make_float2(x, y); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float x, float y) { *(__nv_bfloat162*)p = __floats2bfloat162_rn(x, y); }

constexpr int RGLRU_STAGE = 16, RGLRU_PAIR_THREADS = 32;
template <typename T>
__global__ void __launch_bounds__(RGLRU_PAIR_THREADS)
rglru_scan_pairs_kernel(const float* __restrict__ gates, const T* __restrict__ y, float* __restrict__ state,
                        const int* __restrict__ seg, T* __restrict__ out, int W, int bw) {
  fz_grid_launch_dependents();
  using P = typename PairOf<T>::type;
  constexpr int NST = sizeof(P) == 8 ? 3 : 4;      // stages of the ring (what fits in 48 KB of shared memory)
  __shared__ __align__(16) float2 sa[NST][RGLRU_STAGE][RGLRU_PAIR_THREADS], sb[NST][RGLRU_STAGE][RGLRU_PAIR_THREADS];
  __shared__ __align__(16) P sy[NST][RGLRU_STAGE][RGLRU_PAIR_THREADS];
  const int s = blockIdx.x, tid = threadIdx.x;
  const int c = 2 * (blockIdx.y * RGLRU_PAIR_THREADS + tid);
  const int row0 = seg[4 * s], cnt = seg[4 * s + 1], slot = seg[4 * s + 3];
  fz_grid_wait();
  if (c >= W || cnt <= 0 || slot < 0) return;
  const int part = c / bw, gcol = part * 2 * bw + (c - part * bw);
  // (pointers walk from token to token by a fixed stride; a stage that lies wholly inside the portion has no tests)
  const size_t g_step = (size_t)2 * W, y_step = (size_t)W;
  const float* g_next = gates + (size_t)row0 * g_step + gcol;
  const T* y_next = y + (size_t)row0 * y_step + c;
  int t_next = 0;
  auto issue = [&](int st) {
    if (t_next + RGLRU_STAGE <= cnt) {
#pragma unroll
      for (int i = 0; i < RGLRU_STAGE; ++i) {
        cp_async8(&sa[st][i][tid], g_next + i * g_step);
        cp_async8(&sb[st][i][tid], g_next + i * g_step + bw);
        if (sizeof(P) == 8) cp_async8(&sy[st][i][tid], y_next + i * y_step);
        else cp_async4(&sy[st][i][tid], y_next + i * y_step);
      }
    } else {
      for (int i = 0; t_next + i < cnt; ++i) {
        cp_async8(&sa[st][i][tid], g_next + i * g_step);
        cp_async8(&sb[st][i][tid], g_next + i * g_step + bw);
        if (sizeof(P) == 8) cp_async8(&sy[st][i][tid], y_next + i * y_step);
        else cp_async4(&sy[st][i][tid], y_next + i * y_step);
      }
    }
    cp_async_commit();                       // (past the portion's end: an empty group)
    t_next += RGLRU_STAGE;
    g_next += RGLRU_STAGE * g_step;
    y_next += RGLRU_STAGE * y_step;
  };
  float S0 = state[(size_t)slot * W + c], S1 = state[(size_t)slot * W + c + 1];
#pragma unroll
  for (int k = 0; k < NST - 1; ++k) issue(k);
  int st = 0;
  T* o = out + (size_t)row0 * y_step + c;
  for (int t0 = 0; t0 < cnt; t0 += RGLRU_STAGE, st = st + 1 == NST ? 0 : st + 1, o += RGLRU_STAGE * y_step) {
    issue(st == 0 ? NST - 1 : st - 1);
    cp_async_wait_n<NST - 1>();              // this stage's group has landed
    if (t0 + RGLRU_STAGE <= cnt) {
#pragma unroll
      for (int i = 0; i < RGLRU_STAGE; ++i) {
        const float2 a = sa[st][i][tid], b = sb[st][i][tid], yy = PairOf<T>::f(sy[st][i][tid]);
        S0 = __fmaf_rn(a.x, S0, b.x);
        S1 = __fmaf_rn(a.y, S1, b.y);
        store_pair(o + i * y_step, __fmul_rn(S0, yy.x), __fmul_rn(S1, yy.y));
      }
    } else {
      for (int i = 0; t0 + i < cnt; ++i) {
        const float2 a = sa[st][i][tid], b = sb[st][i][tid], yy = PairOf<T>::f(sy[st][i][tid]);
        S0 = __fmaf_rn(a.x, S0, b.x);
        S1 = __fmaf_rn(a.y, S1, b.y);
        store_pair(o + i * y_step, __fmul_rn(S0, yy.x), __fmul_rn(S1, yy.y));
      }
    }
  }
  state[(size_t)slot * W + c] = S0;
  state[(size_t)slot * W + c + 1] = S1;
}

struct Terms {
  const float* t[4];
  float w[4];
  int n;
};
__global__ void __launch_bounds__(256) weighted_sum_kernel(const Terms p, float* __restrict__ out, size_t total) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float acc = __fmul_rn(p.w[0], p.t[0][i]);
    for (int k = 1; k < p.n; ++k) acc = __fadd_rn(acc, __fmul_rn(p.w[k], p.t[k][i]));
    out[i] = acc;
  }
}

int lanes_per_column(int dk) {
  int R = 1;
  while (R * DPT < dk) R <<= 1;
  return R;
}

size_t attn_smem(int dk, int dv, int pairs) {
  return sizeof(float) * ((size_t)CHUNK * (dk + 1) + (size_t)CHUNK * dv + (size_t)pairs * dk);
}

template <typename K>
int allow_smem(K kern, size_t smem, size_t& allowed) {
  if (smem > allowed) {
    if (smem > 227 * 1024) return FZ_TOO_LARGE;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  return FZ_OK;
}

// rows_per_block: as many rows of a portion as give 32 (row, head) pairs at most.
template <typename T, int DPL>
int launch_sink(AttnArgs a, int N, int n_seg, int max_portion, int units, cudaStream_t stream) {
  const int G_all = a.Hq / a.Hkv, slices = (G_all + MAX_PAIRS - 1) / MAX_PAIRS;
  const int G = G_all < MAX_PAIRS ? G_all : MAX_PAIRS;
  if (units > 0) {                      // single tokens: runs of chunks per block, then the merge
    static size_t allowed_u = 48 * 1024;
    const size_t smem = attn_smem(a.dk, a.dv, G);
    int st = allow_smem(sink_attention_unit_kernel<T, DPL>, smem, allowed_u);
    if (st != FZ_OK) return st;
    fz_launch(sink_attention_unit_kernel<T, DPL>, dim3(N, a.Hkv * slices, units), dim3(32 * ATT_WARPS), smem, stream, a);
    FZ_LAUNCH_CHECK();
    fz_launch(sink_attention_merge_kernel<T, DPL>, dim3(N, a.Hq), dim3(32 * MERGE_WARPS), 0, stream, a);
    FZ_LAUNCH_CHECK();
    return FZ_OK;
  }
  a.rows_per_block = MAX_PAIRS / G > 0 ? MAX_PAIRS / G : 1;
  static size_t allowed_t = 48 * 1024;
  const size_t smem = attn_smem(a.dk, a.dv, a.rows_per_block * G);
  int st = allow_smem(sink_attention_tile_kernel<T, DPL>, smem, allowed_t);
  if (st != FZ_OK) return st;
  const int tiles = (max_portion + a.rows_per_block - 1) / a.rows_per_block;
  if (tiles > 65535 || a.Hkv * slices > 65535) return FZ_TOO_LARGE;
  fz_launch(sink_attention_tile_kernel<T, DPL>, dim3(n_seg + 1, tiles, a.Hkv * slices), dim3(32 * ATT_WARPS), smem, stream, a);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

template <typename T>
int dispatch_sink(const AttnArgs& a, int N, int n_seg, int max_portion, int units, cudaStream_t stream) {
#define FZ_GO(D) return launch_sink<T, D>(a, N, n_seg, max_portion, units, stream)
  const int dpl = (a.dv + 31) / 32;
  if (dpl <= 1) FZ_GO(1);
  if (dpl <= 2) FZ_GO(2);
  if (dpl <= 4) FZ_GO(4);
  if (dpl <= 8) FZ_GO(8);
  if (dpl <= 16) FZ_GO(16);
#undef FZ_GO
  return FZ_BAD_SHAPE;
}
}  // namespace

FZ_API int fz_rotate_kv_write(const float* qkv, int ld, const float* cos_t, const float* sin_t, int rotated, int pairing, int max_pos,
                              const int* pos, const int* seq_row, const int* table, int mb, void* k_pool, void* v_pool,
                              long long page_stride, long long head_stride, long long tok_stride, int page_size,
                              int n_pages, int write, void* q_out, int dtype, int N, int Hq, int Hkv, int dk, int dv,
                              const float* qn_w, const float* kn_w, float norm_eps, float qt_coef, int qt_every, int* err,
                              cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (rotated < 0 || rotated > dk || (rotated & 1) || page_size <= 0 || Hq <= 0 || Hkv <= 0 || dk <= 0 || dv <= 0 ||
      ld < (write ? (Hq + Hkv) * dk + Hkv * dv : Hq * dk) || qt_every < 0 || (write && (qn_w == nullptr) != (kn_w == nullptr)))
    return FZ_BAD_SHAPE;
  const size_t smem = sizeof(float) * (size_t)(Hq + Hkv);
  if (smem > 48 * 1024) return FZ_BAD_SHAPE;
  if (dtype == FZ_F32)
    fz_launch(rotate_kv_write_kernel<float>, dim3(N), dim3(256), smem, stream, qkv, ld, cos_t, sin_t, rotated, pairing, max_pos, pos,
              seq_row, table, mb, (float*)k_pool, (float*)v_pool, page_stride, head_stride, tok_stride, page_size, n_pages,
              write, (float*)q_out, Hq, Hkv, dk, dv, qn_w, kn_w, norm_eps, qt_coef, qt_every, err);
  else if (dtype == FZ_BF16)
    fz_launch(rotate_kv_write_kernel<__nv_bfloat16>, dim3(N), dim3(256), smem, stream, qkv, ld, cos_t, sin_t, rotated, pairing, max_pos,
              pos, seq_row, table, mb, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_stride, head_stride, tok_stride,
              page_size, n_pages, write, (__nv_bfloat16*)q_out, Hq, Hkv, dk, dv, qn_w, kn_w, norm_eps, qt_coef, qt_every, err);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// Sizes taken: Hq any multiple of Hkv, 0 < dk, dv <= 512.
FZ_API int fz_sink_attention_check(int Hq, int Hkv, int dk, int dv) {
  if (Hq <= 0 || Hkv <= 0 || dk <= 0 || dv <= 0 || Hq % Hkv || dk > 512 || dv > 512 || Hkv > 65535) return FZ_BAD_SHAPE;
  return FZ_OK;
}

// How many runs of `unit_chunks` chunks a row can have at most, for contexts up to max_context.
FZ_API int fz_sink_attention_units(int window, int keep_first, int max_context, int unit_chunks, int span) {
  int keys = window > 0 ? (window < max_context ? window : max_context) : max_context;
  if (span > 0 && span < keys) keys = span;
  const int kept = window > 0 ? (keep_first < max_context ? keep_first : max_context) : 0;
  const int chunks = (keys + CHUNK - 1) / CHUNK + 1 + (kept + CHUNK - 1) / CHUNK;
  return (chunks + unit_chunks - 1) / unit_chunks;
}

// Portions are rows of `seg` (n_seg of them, max_portion rows at most). units > 0 (every portion a single token): the
// keys of a row are cut into runs of unit_chunks chunks, `units` at most, with `part` of N * Hq * units * (dv + 2) floats.
FZ_API int fz_sink_attention(const void* q, const void* k_pool, const void* v_pool, const int* pos, const int* seq_row,
                             const int* seg, int n_seg, int max_portion, const int* table, int mb, long long page_stride,
                             long long head_stride, long long tok_stride, int page_size, int n_pages, void* out, int dtype,
                             int N, int Hq, int Hkv, int dk, int dv, float scale, int window, int keep_first,
                             const float* sink, int unit_chunks, int units, float* part, float softcap, const float* gate,
                             int gate_ld, int gate_off, int span, int* err, cudaStream_t stream) {
  if (N <= 0 || n_seg <= 0) return FZ_OK;
  if (span < 0 || (span > 0 && keep_first > 0)) return FZ_BAD_SHAPE;
  if (softcap < 0.f || (gate != nullptr && (gate_off < 0 || gate_off + Hq > gate_ld))) return FZ_BAD_SHAPE;
  if (fz_sink_attention_check(Hq, Hkv, dk, dv) != FZ_OK || page_size <= 0 || window < 0 || keep_first < 0 || max_portion <= 0 ||
      (units > 0 && (unit_chunks <= 0 || part == nullptr || units > 65535))) return FZ_BAD_SHAPE;
  AttnArgs a = {q, k_pool, v_pool, pos, seq_row, seg, table, mb, page_stride, head_stride, tok_stride, page_size, n_pages, out,
                Hq, Hkv, dk, dv, scale, window, keep_first, sink, err, N, 1, unit_chunks, units, part, softcap, gate, gate_ld, gate_off, span};
  if (dtype == FZ_F32) return dispatch_sink<float>(a, N, n_seg, max_portion, units, stream);
  if (dtype == FZ_BF16) return dispatch_sink<__nv_bfloat16>(a, N, n_seg, max_portion, units, stream);
  return FZ_BAD_DTYPE;
}

// The padded key size of the recurrent state, (slots, heads, value_dim, this): 8 times a power of two, at most 256.
FZ_API int fz_recurrent_key_pad(int dk) {
  if (dk <= 0 || dk > 32 * DPT) return -1;
  return lanes_per_column(dk) * DPT;
}

// Shared memory of a scan with `tch` tokens per chunk (floats): what the recurrence reads, then the raw staging area.
// Threads of a scan block: R lanes for each group of DC of the head's value columns, a multiple of 32, SCAN_MAX_THREADS at most.
static int scan_threads(int dv, int R) {
  const long long want = ((long long)((dv + DC - 1) / DC) * R + 31) / 32 * 32;
  return (int)(want < SCAN_MAX_THREADS ? want : SCAN_MAX_THREADS);
}
static size_t retention_smem(int dk, int R, int cols, int rotated, int tch) {
  const int dkp = R * DPT;
  return sizeof(float) * (size_t)tch * ((size_t)2 * dkp + cols + 2 * dk + cols + rotated);
}
static size_t delta_smem(int dk, int R, int cols, int tch, size_t elem) {
  const int dkp = R * DPT;
  return sizeof(float) * (size_t)tch * ((size_t)3 * dkp + cols + 1 + dk + 1) + elem * (size_t)tch * (2 * ((dk + 1) & ~1) + ((cols + 1) & ~1)) + 16;
}

template <int R>
static int launch_retention(const float* proj, int ld, int H, int dk, int dv, const float* decay, float key_scale,
                            const float* cos_t, const float* sin_t, int rotated, int pairing, int max_pos, float* state,
                            const int* seg, int n_seg, float* out, int* err, cudaStream_t stream) {
  const int threads = scan_threads(dv, R), cols = threads / R * DC;
  const int tch = retention_smem(dk, R, cols, rotated, 16) <= 48 * 1024 ? 16 : 8;
  const size_t smem = retention_smem(dk, R, cols, rotated, tch);
  static size_t allowed = 48 * 1024;
  int st = allow_smem(retention_scan_kernel<R>, smem, allowed);
  if (st != FZ_OK) return st;
  fz_launch(retention_scan_kernel<R>, dim3(n_seg, H, (dv + cols - 1) / cols), dim3(threads), smem, stream, proj, ld, H, dk, dv,
            tch, decay, key_scale, cos_t, sin_t, rotated, pairing, max_pos, state, seg, out, err);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

#define FZ_BY_LANES(R, CALL)          \
  switch (R) {                        \
    case 1: return CALL(1);           \
    case 2: return CALL(2);           \
    case 4: return CALL(4);           \
    case 8: return CALL(8);           \
    case 16: return CALL(16);         \
    default: return CALL(32);         \
  }

FZ_API int fz_retention_scan(const float* proj, int ld, int H, int dk, int dv, const float* decay, float key_scale,
                             const float* cos_t, const float* sin_t, int rotated, int pairing, int max_pos, float* state,
                             const int* seg, int n_seg, float* out, int* err, cudaStream_t stream) {
  if (n_seg <= 0) return FZ_OK;
  if (H <= 0 || H > 65535 || dv <= 0 || fz_recurrent_key_pad(dk) < 0 || rotated < 0 || rotated > dk || (rotated & 1)) return FZ_BAD_SHAPE;
#define FZ_CALL(R) launch_retention<R>(proj, ld, H, dk, dv, decay, key_scale, cos_t, sin_t, rotated, pairing, max_pos, state, seg, n_seg, out, err, stream)
  FZ_BY_LANES(lanes_per_column(dk), FZ_CALL)
#undef FZ_CALL
}

template <typename T, int R>
static int launch_delta(const void* qkv, int H, int Hk, int dk, int dv, const float* high, int ldh, const float* beta,
                        const float* a_log, const float* dt_bias, float unit_eps, float q_scale, float* state, const int* seg,
                        int n_seg, float* out, cudaStream_t stream) {
  const int threads = scan_threads(dv, R), cols = threads / R * DC;
  const int tch = delta_smem(dk, R, cols, 16, sizeof(T)) <= 48 * 1024 ? 16 : 8;
  const size_t smem = delta_smem(dk, R, cols, tch, sizeof(T));
  static size_t allowed = 48 * 1024;
  int st = allow_smem(gated_delta_scan_kernel<T, R>, smem, allowed);
  if (st != FZ_OK) return st;
  fz_launch(gated_delta_scan_kernel<T, R>, dim3(n_seg, H, (dv + cols - 1) / cols), dim3(threads), smem, stream, (const T*)qkv,
            H, Hk, dk, dv, tch, high, ldh, beta, a_log, dt_bias, unit_eps, q_scale, state, seg, out);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_gated_delta_scan(const void* qkv, int dtype, int H, int Hk, int dk, int dv, const float* high, int ldh,
                               const float* beta, const float* a_log, const float* dt_bias, float unit_eps, float q_scale,
                               float* state, const int* seg, int n_seg, float* out, cudaStream_t stream) {
  if (n_seg <= 0) return FZ_OK;
  if (H <= 0 || H > 65535 || Hk <= 0 || H % Hk || dv <= 0 || fz_recurrent_key_pad(dk) < 0) return FZ_BAD_SHAPE;
#define FZ_CALL_F(R) launch_delta<float, R>(qkv, H, Hk, dk, dv, high, ldh, beta, a_log, dt_bias, unit_eps, q_scale, state, seg, n_seg, out, stream)
#define FZ_CALL_B(R) launch_delta<__nv_bfloat16, R>(qkv, H, Hk, dk, dv, high, ldh, beta, a_log, dt_bias, unit_eps, q_scale, state, seg, n_seg, out, stream)
  if (dtype == FZ_F32) { FZ_BY_LANES(lanes_per_column(dk), FZ_CALL_F) }
  if (dtype == FZ_BF16) { FZ_BY_LANES(lanes_per_column(dk), FZ_CALL_B) }
#undef FZ_CALL_F
#undef FZ_CALL_B
  return FZ_BAD_DTYPE;
}

static size_t general_delta_smem(int dk, int R, int cols, int tch) {
  const int dkp = R * DPT;
  return sizeof(float) * (size_t)tch * ((size_t)5 * dkp + cols + 4 * dk + cols);
}

template <int R>
static int launch_general_delta(const float* proj, int ld, int H, int dk, int dv, int off_a, const float* din, const float* dbias,
                                const float* abias, float rate, float unit_eps, float* state, const int* seg, int n_seg,
                                float* out, cudaStream_t stream) {
  const int threads = scan_threads(dv, R), cols = threads / R * DC;
  const int tch = general_delta_smem(dk, R, cols, 16) <= 48 * 1024 ? 16 : 8;
  const size_t smem = general_delta_smem(dk, R, cols, tch);
  static size_t allowed = 48 * 1024;
  int st = allow_smem(general_delta_scan_kernel<R>, smem, allowed);
  if (st != FZ_OK) return st;
  fz_launch(general_delta_scan_kernel<R>, dim3(n_seg, H, (dv + cols - 1) / cols), dim3(threads), smem, stream, proj, ld, H, dk,
            dv, off_a, tch, din, dbias, abias, rate, unit_eps, state, seg, out);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_general_delta_scan(const float* proj, int ld, int H, int dk, int dv, int off_a, const float* din,
                                 const float* dbias, const float* abias, float rate, float unit_eps, float* state,
                                 const int* seg, int n_seg, float* out, cudaStream_t stream) {
  if (n_seg <= 0) return FZ_OK;
  if (H <= 0 || H > 65535 || dv <= 0 || fz_recurrent_key_pad(dk) < 0 || ld < 2 * H * dk + H * dv || off_a < 0 || off_a + H * dk > ld)
    return FZ_BAD_SHAPE;
#define FZ_CALL(R) launch_general_delta<R>(proj, ld, H, dk, dv, off_a, din, dbias, abias, rate, unit_eps, state, seg, n_seg, out, stream)
  FZ_BY_LANES(lanes_per_column(dk), FZ_CALL)
#undef FZ_CALL
}

// act: 0 none, 1 sigmoid, 2 silu.
// w: dv values shared by the heads, or (w_per_head) H * dv values.
FZ_API int fz_head_norm_gate(const float* o, int N, int H, int dv, const float* w, int w_per_head, float eps, const float* gate, int ldg,
                             int goff, int act, const int* seq_row, void* out, int out_dtype, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (H <= 0 || dv <= 0) return FZ_BAD_SHAPE;
  const int W = H < 8 ? H : 8;
  if (out_dtype == FZ_F32)
    fz_launch(head_norm_gate_kernel<float>, dim3(N), dim3(32 * W), 0, stream, o, H, dv, w, w_per_head, eps, gate, ldg, goff, act, seq_row, (float*)out);
  else if (out_dtype == FZ_BF16)
    fz_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(N), dim3(32 * W), 0, stream, o, H, dv, w, w_per_head, eps, gate, ldg, goff, act, seq_row, (__nv_bfloat16*)out);
  else return FZ_BAD_DTYPE;
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_router_topk(const float* logits, int ld, int N, int E, int top, int groups, int keep, int renorm,
                          const int* seq_row, int* choice, float* weight, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (E <= 0 || E > 2048 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > keep * (E / groups)) return FZ_BAD_SHAPE;
  const size_t smem = sizeof(float) * ROUTER_WARPS * (size_t)(E + groups + top);
  fz_launch(router_topk_kernel, dim3((N + ROUTER_WARPS - 1) / ROUTER_WARPS), dim3(32 * ROUTER_WARPS), smem, stream, logits, ld,
            N, E, top, groups, keep, renorm, seq_row, choice, weight);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_moe_combine(const float* terms, const float* w, int top, const float* shared, const float* gl, int ldg, int col,
                          const int* seq_row, float* out, int N, int D, const float* add, float scale, cudaStream_t stream) {
  if (N <= 0 || D <= 0) return FZ_OK;
  const int by = (D + 1023) / 1024 > 0 ? (D + 1023) / 1024 : 1;
  fz_launch(moe_combine_kernel, dim3(N, by), dim3(256), 0, stream, terms, w, top, shared, gl, ldg, col, seq_row, out, N, D, add,
            scale);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

// cooked != 0: two launches (the gate inputs are overwritten by the recurrence's coefficients); else the scan alone.
FZ_API int fz_rglru_scan(const void* u, float* gates, const float* gbias, const float* lam, const void* y, float sharp,
                         float* state, const int* seg, int n_seg, const int* seq_row, void* out, int dtype, int N, int W, int B,
                         int cooked, cudaStream_t stream) {
  if (N <= 0 || n_seg <= 0) return FZ_OK;
  if (W <= 0 || B <= 0 || W % B || n_seg > 65535 * 32) return FZ_BAD_SHAPE;
  if (dtype != FZ_F32 && dtype != FZ_BF16) return FZ_BAD_DTYPE;
  const int bw = W / B;
  // long portions (few of them in a step): blocks of 32 or 16 channels until the channels alone fill the SMs
  int tpb = 64;
  while (cooked && tpb > 16 && (W + tpb - 1) / tpb < 148) tpb >>= 1;
  const dim3 grid(n_seg, (W + tpb - 1) / tpb);
  if (cooked) {
    const long long total = (long long)N * W;
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    if (dtype == FZ_F32)
      fz_launch(rglru_cook_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (const float*)u, gates, gbias, lam, sharp, seq_row, W, bw, total);
    else
      fz_launch(rglru_cook_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)u, gates, gbias, lam, sharp, seq_row, W, bw, total);
    FZ_LAUNCH_CHECK();
    if (W % 2 == 0 && bw % 2 == 0 && (((uintptr_t)gates | (uintptr_t)y | (uintptr_t)out) & 15) == 0) {
      const dim3 pgrid(n_seg, (W / 2 + RGLRU_PAIR_THREADS - 1) / RGLRU_PAIR_THREADS);
      if (dtype == FZ_F32)
        fz_launch(rglru_scan_pairs_kernel<float>, pgrid, dim3(RGLRU_PAIR_THREADS), 0, stream, gates, (const float*)y, state, seg, (float*)out, W, bw);
      else
        fz_launch(rglru_scan_pairs_kernel<__nv_bfloat16>, pgrid, dim3(RGLRU_PAIR_THREADS), 0, stream, gates, (const __nv_bfloat16*)y, state, seg,
                  (__nv_bfloat16*)out, W, bw);
      FZ_LAUNCH_CHECK();
      return FZ_OK;
    }
    if (dtype == FZ_F32)
      fz_launch(rglru_scan_kernel<float, true>, grid, dim3(tpb), 0, stream, (const float*)u, gates, gbias, lam, (const float*)y, sharp, state, seg, (float*)out, W, bw);
    else
      fz_launch(rglru_scan_kernel<__nv_bfloat16, true>, grid, dim3(tpb), 0, stream, (const __nv_bfloat16*)u, gates, gbias, lam, (const __nv_bfloat16*)y, sharp, state, seg, (__nv_bfloat16*)out, W, bw);
  } else {
    if (dtype == FZ_F32)
      fz_launch(rglru_scan_kernel<float, false>, grid, dim3(64), 0, stream, (const float*)u, gates, gbias, lam, (const float*)y, sharp, state, seg, (float*)out, W, bw);
    else
      fz_launch(rglru_scan_kernel<__nv_bfloat16, false>, grid, dim3(64), 0, stream, (const __nv_bfloat16*)u, gates, gbias, lam, (const __nv_bfloat16*)y, sharp, state, seg, (__nv_bfloat16*)out, W, bw);
  }
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

FZ_API int fz_weighted_sum(const float* t0, const float* t1, const float* t2, const float* t3, float w0, float w1, float w2,
                           float w3, int n_terms, float* out, long long total, cudaStream_t stream) {
  if (total <= 0) return FZ_OK;
  if (n_terms < 1 || n_terms > 4) return FZ_BAD_SHAPE;
  Terms p = {{t0, t1, t2, t3}, {w0, w1, w2, w3}, n_terms};
  const long long blocks = (total + 255) / 256;
  fz_launch(weighted_sum_kernel, dim3((unsigned)(blocks < 65535 ? blocks : 65535)), dim3(256), 0, stream, p, out, (size_t)total);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(seq_mix)
#endif
