// Attention over a sliding window that keeps the first tokens, with a sink in the softmax, for prompt portions over the
// paged bf16 cache, on tensor cores (mma.sync m16n8k16): key and value size 64 or 128.
//
// grid (portions + 1, tiles of 64 rows of a portion, query heads), 128 threads; warp w owns rows 16 w .. 16 w + 15 of its
// tile. Key tiles of 64 start at multiples of 64 in absolute position: first the tiles of the kept first tokens that
// lie before the tile's window, then the window's up to the tile's last row's own position, through a two-stage
// cp.async ring; S = Q K^T and O += P V accumulate in float32, softmax is online in the exp2 domain with float32 max
// and sum, P is rounded to bf16 for the second product; a row sees key j if j <= p and (p - j < window or j <
// keep_first); the sink (a learned number per head, not scaled) joins the denominator at the end. The block after the
// last portion's writes zeros into the rows of padding.
#include "attn_mma.cuh"
#include <math.h>

namespace {
using namespace fzattn;

constexpr int BM = 64, BN = 64, THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

template <int HD>
__global__ void __launch_bounds__(THREADS)
sink_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                          const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ seg,
                          const int* __restrict__ seq_row, const int* __restrict__ table, int mb, long long page_stride,
                          long long head_stride, long long tok_stride, int page_size, int n_pages,
                          __nv_bfloat16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window, int keep_first,
                          const float* __restrict__ sink, float cap_log2, float over_cap, const float* __restrict__ gate,
                          int gate_ld, int gate_off, int N, int* err, int span) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  constexpr int KSTEPS = HD / 16, NB = HD / 8, TILE_BYTES = BN * HD * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s_base = smem_u32(smem);          // [2 stages][K | V], then Q
  const uint32_t s_q = s_base + 4 * TILE_BYTES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // grid (portions + 1, heads, row tiles): blocks are handed out with the tile index falling, so a portion's last
  // tiles, which have the most keys behind them under a causal or chunked mask, start first and the short ones fill
  // the tail
  const int h = blockIdx.y, tile = (int)(gridDim.z - 1 - blockIdx.z);
  if (blockIdx.x == gridDim.x - 1) {               // rows of padding get zeros
    if (tile == 0)
      for (int n = 0; n < N; ++n)
        if (seq_row[n] < 0)
          for (int i = tid; i < HD; i += THREADS) out[((size_t)n * Hq + h) * HD + i] = __float2bfloat16_rn(0.f);
    return;
  }
  const int s_idx = blockIdx.x, r_off = BM * tile;
  const int row0 = seg[4 * s_idx], n_rows = seg[4 * s_idx + 1], pos0 = seg[4 * s_idx + 2];
  if (r_off >= n_rows) return;
  const int kvh = h / (Hq / Hkv);
  const int valid_rows = min(BM, n_rows - r_off);
  const int qpos0 = pos0 + r_off;                               // position of the tile's first row
  const int last_pos = qpos0 + valid_rows - 1;
  // (span > 0, a chunked mask: a row also sees nothing before the start of its own block of `span` positions)
  const int lo_tile = max(window > 0 ? max(0, qpos0 - window + 1) : 0, span > 0 ? qpos0 - qpos0 % span : 0);
  const int kept = window > 0 ? min(keep_first, lo_tile) : 0;   // keys 0 .. kept-1 are seen although they lie before the window
  const int first_end = kept > 0 ? (kept - 1) / BN : -1;        // last key tile of the kept tokens
  const int c2 = max(lo_tile / BN, first_end + 1);              // first key tile of the window not yet walked
  const int ntiles = first_end + 1 + max(0, last_pos / BN - c2 + 1);
  const int* trow = table + (size_t)seq_row[row0] * mb;
  const long long head_off = (long long)kvh * head_stride;

  {
    const __nv_bfloat16* qbase = q + (size_t)(row0 + r_off) * Hq * HD + (size_t)h * HD;
    for (int e = tid; e < BM * (HD / 8); e += THREADS) {
      const int r = e / (HD / 8), c = e - r * (HD / 8);
      cp_async16(s_q + swz<HD>(r, c), qbase + (size_t)r * Hq * HD + c * 8, r < valid_rows);
    }
  }
  auto key_tile = [&](int it) { return (it <= first_end ? it : c2 + (it - first_end - 1)) * BN; };
  auto issue = [&](int it) {
    const uint32_t sk = s_base + (it & 1) * 2 * TILE_BYTES, sv = sk + TILE_BYTES;
    constexpr int TPR = THREADS / BN, CPT = (HD / 8) / TPR;      // threads per key row, 16-byte chunks per thread
    const int r = tid / TPR, cfirst = (tid % TPR) * CPT;
    const int key = key_tile(it) + r;
    bool valid = key <= last_pos && (key >= lo_tile || key < keep_first);
    long long off = 0;
    if (valid) {
      const int page = trow[key / page_size];
      if (page < 0 || page >= n_pages) { atomicOr(err, FZ_ERR_NO_PAGE); valid = false; }
      else off = (long long)page * page_stride + head_off + (long long)(key % page_size) * tok_stride;
    }
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int c = cfirst + i;
      cp_async16(sk + swz<HD>(r, c), k_pool + off + c * 8, valid);
      cp_async16(sv + swz<HD>(r, c), v_pool + off + c * 8, valid);
    }
    cp_async_commit();
  };
  issue(0);

  uint32_t qf[KSTEPS][4];
  float o[NB][4];
#pragma unroll
  for (int i = 0; i < NB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int r_lo = warp * 16 + (lane >> 2);                     // this thread's rows: r_lo and r_lo + 8
  const int qp[2] = {qpos0 + r_lo, qpos0 + r_lo + 8};
  const int warp_first = qpos0 + warp * 16, warp_last = min(warp_first + 15, last_pos);

  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) { issue(t + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(qf[ks], s_q + swz<HD>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
    }
    const int key0 = key_tile(t);
    // a warp whose rows all lie before this key tile, or whose windows all ended before it (and that is not a tile of
    // kept tokens), has nothing to do here
    const bool active = warp * 16 < valid_rows && key0 <= warp_last &&
                        (window <= 0 || key0 + BN - 1 >= warp_first - window + 1 || key0 < keep_first) &&
                        (span <= 0 || key0 + BN - 1 >= warp_first - warp_first % span);
    if (active) {
      const uint32_t sk = s_base + (t & 1) * 2 * TILE_BYTES, sv = sk + TILE_BYTES;
      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int jb = 0; jb < BN / 16; ++jb) {
          uint32_t kf[4];
          const int mi = lane >> 3;
          ldmatrix_x4(kf, sk + swz<HD>(jb * 16 + (mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1)));
          mma_bf16(s[2 * jb], qf[ks], kf[0], kf[1]);
          mma_bf16(s[2 * jb + 1], qf[ks], kf[2], kf[3]);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + 8 * j + 2 * (lane & 3) + (e & 1);
          const int qpos = qp[e >> 1];
          const bool ok = key <= qpos && (window <= 0 || key >= qpos - window + 1 || key < keep_first) &&
                          (span <= 0 || key >= qpos - qpos % span);
          // (a cap c > 0: the scaled score x becomes c tanh(x / c); cap_log2 = c log2(e), over_cap = scale / c)
          const float x = cap_log2 > 0.f ? cap_log2 * tanhf(s[j][e] * over_cap) : s[j][e] * scale_log2;
          const float v = ok ? x : -INFINITY;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2], mu[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
        const float mn = fmaxf(m_run[hh], mx[hh]);
        mu[hh] = mn == -INFINITY ? 0.f : mn;
        corr[hh] = exp2f(m_run[hh] - mu[hh]);
        m_run[hh] = mn;
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
        s[j][0] = exp2f(s[j][0] - mu[0]); s[j][1] = exp2f(s[j][1] - mu[0]);
        s[j][2] = exp2f(s[j][2] - mu[1]); s[j][3] = exp2f(s[j][3] - mu[1]);
        sum[0] += s[j][0] + s[j][1];
        sum[1] += s[j][2] + s[j][3];
      }
      l_run[0] = l_run[0] * corr[0] + sum[0];
      l_run[1] = l_run[1] * corr[1] + sum[1];
#pragma unroll
      for (int i = 0; i < NB; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {       // 16 keys per k-step
        uint32_t pf[4];
        pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
          uint32_t vf[4];
          const int mi = lane >> 3;
          ldmatrix_x4_trans(vf, sv + swz<HD>(kk * 16 + (mi & 1) * 8 + (lane & 7), nb + (mi >> 1)));
          mma_bf16(o[nb], pf, vf[0], vf[1]);
          mma_bf16(o[nb + 1], pf, vf[2], vf[3]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = r_lo + 8 * hh;
    if (r >= valid_rows) continue;
    float l = l_run[hh], corr = 1.f;
    if (sink != nullptr) {                         // one more term of the denominator, no value
      const float sk2 = sink[h] * LOG2E;
      const float mn = fmaxf(m_run[hh], sk2);
      corr = exp2f(m_run[hh] - mn);
      l = l * corr + exp2f(sk2 - mn);
    }
    float inv = corr / l;
    if (gate != nullptr)                           // a gate per head: the result times its sigmoid
      inv *= 1.0f / (1.0f + expf(-gate[(size_t)(row0 + r_off + r) * gate_ld + gate_off + h]));
    __nv_bfloat16* orow = out + (size_t)(row0 + r_off + r) * Hq * HD + (size_t)h * HD + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < NB; ++i)
      *(uint32_t*)(orow + 8 * i) = pack_bf16(o[i][2 * hh] * inv, o[i][2 * hh + 1] * inv);
  }
}

template <int HD>
int launch(const void* q, const void* k_pool, const void* v_pool, const int* seg, const int* seq_row, int n_seg, int max_portion,
           const int* table, int mb, long long page_stride, long long head_stride, long long tok_stride, int page_size,
           int n_pages, void* out, int N, int Hq, int Hkv, float scale, int window, int keep_first, const float* sink,
           float softcap, const float* gate, int gate_ld, int gate_off, int span, int* err, cudaStream_t stream) {
  constexpr size_t smem = 4 * (BN * HD * 2) + BM * HD * 2;
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaError_t e = cudaFuncSetAttribute(sink_attention_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  const int tiles = (max_portion + BM - 1) / BM;
  if (tiles > 65535 || Hq > 65535) return FZ_TOO_LARGE;
  fz_launch(sink_attention_mma_kernel<HD>, dim3(n_seg + 1, Hq, tiles), dim3(THREADS), smem, stream, (const __nv_bfloat16*)q,
            (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, seg, seq_row, table, mb, page_stride, head_stride,
            tok_stride, page_size, n_pages, (__nv_bfloat16*)out, Hq, Hkv, scale * LOG2E, window, keep_first, sink,
            softcap > 0.f ? softcap * LOG2E : 0.f, softcap > 0.f ? scale / softcap : 0.f, gate, gate_ld, gate_off, N, err,
            span);
  FZ_LAUNCH_CHECK();
  return FZ_OK;
}
}  // namespace

// Sizes taken: keys and values of one size, 64 or 128; strides of the pools that keep every row 16-byte aligned.
FZ_API int fz_sink_attention_mma_check(int Hq, int Hkv, int dk, int dv, const void* k_pool, const void* v_pool,
                                       long long page_stride, long long head_stride, long long tok_stride) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || dk != dv || (dk != 64 && dk != 128)) return FZ_BAD_SHAPE;
  if ((page_stride | head_stride | tok_stride) & 7 || ((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return FZ_BAD_ALIGNMENT;
  return FZ_OK;
}

FZ_API int fz_sink_attention_mma(const void* q, const void* k_pool, const void* v_pool, const int* seg, const int* seq_row,
                                 int n_seg, int max_portion, const int* table, int mb, long long page_stride,
                                 long long head_stride, long long tok_stride, int page_size, int n_pages, void* out, int N,
                                 int Hq, int Hkv, int hd, float scale, int window, int keep_first, const float* sink,
                                 float softcap, const float* gate, int gate_ld, int gate_off, int span, int* err,
                                 cudaStream_t stream) {
  if (N <= 0 || n_seg <= 0) return FZ_OK;
  if (span < 0 || (span > 0 && keep_first > 0)) return FZ_BAD_SHAPE;
  if (softcap < 0.f || (gate != nullptr && (gate_off < 0 || gate_off + Hq > gate_ld))) return FZ_BAD_SHAPE;
  if (fz_sink_attention_mma_check(Hq, Hkv, hd, hd, k_pool, v_pool, page_stride, head_stride, tok_stride) != FZ_OK ||
      page_size <= 0 || max_portion <= 0 || window < 0 || keep_first < 0 || ((uintptr_t)q & 15)) return FZ_BAD_SHAPE;
  if (hd == 64)
    return launch<64>(q, k_pool, v_pool, seg, seq_row, n_seg, max_portion, table, mb, page_stride, head_stride, tok_stride,
                      page_size, n_pages, out, N, Hq, Hkv, scale, window, keep_first, sink, softcap, gate, gate_ld, gate_off, span, err, stream);
  return launch<128>(q, k_pool, v_pool, seg, seq_row, n_seg, max_portion, table, mb, page_stride, head_stride, tok_stride,
                     page_size, n_pages, out, N, Hq, Hkv, scale, window, keep_first, sink, softcap, gate, gate_ld, gate_off, span, err, stream);
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(attn_sink_mma)
#endif
