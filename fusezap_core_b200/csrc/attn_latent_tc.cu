// Attention over a paged cache of one bf16 vector per token shared by all heads, on tensor cores: prompt portions and
// decoded tokens in one kernel.
//
// Because every head reads the same cached vectors, the (token row, head) pairs of a portion are the rows of ONE
// attention problem: q is (N, H, W) contiguous, so the pairs of a portion are consecutive rows of W values, and pair p
// of the portion sits at position pos0 + p / H. A block takes 64 consecutive pairs of one portion (for a decoded token:
// its H heads) and walks the request's keys in tiles of BN, two cp.async stages. Eight warps: warp w serves the 16 pairs
// 16 (w & 3) ..; for S = Q E^T the two warps of a pair group split the tile's keys, for O += P E[:, :Wv] they split the
// value columns, so P goes through shared memory (bf16, as the other attention kernels round it) and a thread holds
// Wv / 8 accumulators. mma.sync m16n8k16, float32 scores, online softmax in the exp2 domain with float32 max and sum.
// Key tiles start at multiples of BN in absolute position, so a row's sums do not depend on how the prompt was cut.
//
// With `sink` (one float32 per head) the denominator of pair p, head p % H, also holds exp(sink): it enters once, in the
// epilogue, or in the merge kernel where the keys were cut into ranges.
//
// Sizes: W % 16 == 0, W <= 1024; value width Wv <= W, padded to a multiple of 32 that still fits in W (the padded
// columns are computed and not stored). Everything else goes to the general kernel.
#include "attn_mma.cuh"
#include <math.h>

namespace {
using namespace fzattn;

constexpr int BM = 64, THREADS = 256, PAD = 8;

// Rows of `stride` bf16 (W + 8: consecutive rows start 16 bytes further along the banks, so the eight rows of an
// ldmatrix never collide); chunk c is the row's c-th group of eight values.
__device__ __forceinline__ uint32_t at(uint32_t base, int row, int chunk, int stride) {
  return base + (uint32_t)(row * stride * 2 + chunk * 16);
}

// Which portion holds tile `tile` (tiles are numbered portion by portion, ceil(rows * H / 64) each), and the tile's first
// pair within it. Every warp works it out for itself: 32 portions per round, a lane loads one portion's row count, a
// prefix sum over the lanes, a ballot for the first portion whose tiles reach past `tile`. Returns -1 if there is none.
__device__ __forceinline__ int locate_tile(const int* __restrict__ seg, int n_seg, int H, int tile, int& pair0) {
  const int lane = threadIdx.x & 31;
  int base = 0;
  for (int s0 = 0; s0 < n_seg; s0 += 32) {
    const int s = s0 + lane;
    const int mine = s < n_seg ? (seg[4 * s + 1] * H + BM - 1) / BM : 0;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, tile < base + incl);
    if (hit) {
      const int first = __ffs(hit) - 1;
      const int before = base + __shfl_sync(0xffffffffu, incl - mine, first);
      pair0 = (tile - before) * BM;
      return s0 + first;
    }
    base += __shfl_sync(0xffffffffu, incl, 31);
  }
  return -1;
}

template <int NV16, int BN>      // a warp's value columns: NV16 * 16; keys per tile: BN
__global__ void __launch_bounds__(THREADS)
attn_latent_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ pool,
                      const int* __restrict__ seg, int n_seg, const int* __restrict__ table, int mb,
                      long long page_stride, int page_size, int num_pages, __nv_bfloat16* __restrict__ out, int H, int W,
                      int Wv, float scale_log2, int window, float* __restrict__ part_o, float* __restrict__ part_ml,
                      int split_keys, int* err, const float* __restrict__ sink) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  constexpr int NBS = BN / 16;                 // 8-key blocks of S per warp (half the tile's keys)
  const int stride = W + PAD, pstride = BN + PAD;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t s_q = smem_u32(smem);
  const uint32_t s_k = s_q + BM * stride * 2;                   // two stages of [BN][stride]
  const uint32_t s_p = s_k + 2 * BN * stride * 2;               // [BM][pstride]
  float* red = (float*)(smem + (size_t)BM * stride * 2 + (size_t)2 * BN * stride * 2 + (size_t)BM * pstride * 2);   // [2][BM]

  // which portion, and which 64 pairs of it. Blocks are handed out in rising blockIdx.x: the tile index falls with it,
  // so a prompt's last tiles, which have the most keys behind them, start first and the short ones fill the tail.
  const int tile = gridDim.x - 1 - blockIdx.x;
  int pair0 = 0;
  const int s_idx = locate_tile(seg, n_seg, H, tile, pair0);
  if (s_idx < 0) return;
  const int row0 = seg[4 * s_idx], n_rows = seg[4 * s_idx + 1], pos0 = seg[4 * s_idx + 2];
  const int valid = min(BM, n_rows * H - pair0);
  const int first_pos = pos0 + pair0 / H, last_pos = pos0 + (pair0 + valid - 1) / H;
  const int lo_tile = window > 0 ? max(0, first_pos - window + 1) : 0;
  // split_keys > 0: the keys are cut at multiples of split_keys and block (x, y) takes the y-th range; its result stays
  // unnormalised in float32 scratch with the row's (max, sum), for the merge kernel
  const int key_lo = split_keys > 0 ? max(lo_tile, (int)blockIdx.y * split_keys) : lo_tile;
  const int key_hi = split_keys > 0 ? min(last_pos, ((int)blockIdx.y + 1) * split_keys - 1) : last_pos;
  const size_t part = (size_t)tile * gridDim.y + blockIdx.y;
  if (key_lo > key_hi) {      // nothing of this range is visible to the tile (split mode only)
    for (int r = threadIdx.x; r < BM; r += THREADS) {
      part_ml[(part * BM + r) * 2] = -INFINITY;
      part_ml[(part * BM + r) * 2 + 1] = 0.f;
    }
    return;
  }
  const int k_begin = key_lo & ~(BN - 1);
  const int ntiles = (key_hi - k_begin) / BN + 1;
  const int* trow = table + (size_t)s_idx * mb;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, half = warp >> 2;
  const int chunks = W / 8;

  {
    const __nv_bfloat16* qbase = q + ((size_t)row0 * H + pair0) * W;
    for (int e = tid; e < BM * chunks; e += THREADS) {
      const int r = e / chunks, c = e - r * chunks;
      cp_async16(at(s_q, r, c, stride), qbase + (size_t)r * W + c * 8, r < valid);
    }
  }
  // A key row of the tile is copied by THREADS / BN threads, each looking the row's page up once (the lookup is a load
  // from global memory that the copies depend on: one per thread and tile, not one per 16 bytes).
  constexpr int TPR = THREADS / BN;
  const int my_row = tid / TPR, my_sub = tid - my_row * TPR;
  auto issue = [&](int t) {
    const uint32_t st = s_k + (t & 1) * BN * stride * 2;
    const int key = k_begin + t * BN + my_row;
    bool ok = key >= key_lo && key <= key_hi;
    const __nv_bfloat16* src = pool;
    if (ok) {
      const int pi = key / page_size;
      const int page = trow[pi];
      ok = page >= 0 && page < num_pages;
      if (!ok) atomicOr(err, FZ_ERR_NO_PAGE);
      else src = pool + (long long)page * page_stride + (long long)(key - pi * page_size) * W;
    }
    for (int c = my_sub; c < chunks; c += TPR) cp_async16(at(st, my_row, c, stride), ok ? src + c * 8 : pool, ok);
    cp_async_commit();
  };
  issue(0);

  float o[2 * NV16][4];
#pragma unroll
  for (int i = 0; i < 2 * NV16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int r_lo = rg * 16 + (lane >> 2);                        // this thread's pairs: r_lo and r_lo + 8
  const int qp[2] = {pos0 + (pair0 + r_lo) / H, pos0 + (pair0 + r_lo + 8) / H};
  const int ksteps = W / 16;
  // A pair group none of whose 16 pairs exists (a decoded token with few heads, a portion's last tile) takes part in the
  // loads and the barriers only: its products are skipped (the decision is the same for all lanes of a warp).
  const bool active = rg * 16 < valid;

  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) { issue(t + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint32_t sk = s_k + (t & 1) * BN * stride * 2;
    const int key0 = k_begin + t * BN, kh0 = half * (BN / 2);    // this warp's keys of the tile: kh0 .. kh0 + BN/2 - 1
    // two sets of accumulators, for even and odd k-steps: consecutive MMAs do not wait on each other, and with the loop
    // unrolled the loads of the next k-steps are issued under the MMAs of this one
    float s[NBS][4], s2[NBS][4];
#pragma unroll
    for (int j = 0; j < NBS; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; s2[j][0] = s2[j][1] = s2[j][2] = s2[j][3] = 0.f; }
    auto k_step = [&](int ks, float (*acc)[4]) {
      uint32_t qf[4];
      ldmatrix_x4(qf, at(s_q, rg * 16 + (lane & 15), ks * 2 + (lane >> 4), stride));
#pragma unroll
      for (int jb = 0; jb < NBS / 2; ++jb) {
        uint32_t kf[4];
        const int mi = lane >> 3;
        ldmatrix_x4(kf, at(sk, kh0 + jb * 16 + (mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1), stride));
        mma_bf16(acc[2 * jb], qf, kf[0], kf[1]);
        mma_bf16(acc[2 * jb + 1], qf, kf[2], kf[3]);
      }
    };
    if (active) {
      int ks = 0;
#pragma unroll 2
      for (; ks + 1 < ksteps; ks += 2) {
        k_step(ks, s);
        k_step(ks + 1, s2);
      }
      if (ks < ksteps) k_step(ks, s);
    }
#pragma unroll
    for (int j = 0; j < NBS; ++j) { s[j][0] += s2[j][0]; s[j][1] += s2[j][1]; s[j][2] += s2[j][2]; s[j][3] += s2[j][3]; }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NBS; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + kh0 + 8 * j + 2 * (lane & 3) + (e & 1);
        const int qpos = qp[e >> 1];
        const bool ok = key <= qpos && key >= key_lo && key <= key_hi && (window <= 0 || key >= qpos - window + 1);
        const float v = ok ? s[j][e] * scale_log2 : -INFINITY;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
    }
    if ((lane & 3) == 0) {
      red[half * BM + r_lo] = mx[0];
      red[half * BM + r_lo + 8] = mx[1];
    }
    __syncthreads();
    float corr[2], mu[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const float both = fmaxf(red[r_lo + 8 * hh], red[BM + r_lo + 8 * hh]);
      const float mn = fmaxf(m_run[hh], both);
      mu[hh] = mn == -INFINITY ? 0.f : mn;
      corr[hh] = exp2f(m_run[hh] - mu[hh]);
      m_run[hh] = mn;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NBS; ++j) {
      s[j][0] = exp2f(s[j][0] - mu[0]); s[j][1] = exp2f(s[j][1] - mu[0]);
      s[j][2] = exp2f(s[j][2] - mu[1]); s[j][3] = exp2f(s[j][3] - mu[1]);
      sum[0] += s[j][0] + s[j][1];
      sum[1] += s[j][2] + s[j][3];
      // P (bf16) for the second product: row r_lo (+8), keys kh0 + 8 j + 2 (lane & 3) (+1)
      const int col = kh0 + 8 * j + 2 * (lane & 3);
      *(uint32_t*)(smem + (s_p - s_q) + ((size_t)r_lo * pstride + col) * 2) = pack_bf16(s[j][0], s[j][1]);
      *(uint32_t*)(smem + (s_p - s_q) + ((size_t)(r_lo + 8) * pstride + col) * 2) = pack_bf16(s[j][2], s[j][3]);
    }
    l_run[0] = l_run[0] * corr[0] + sum[0];
    l_run[1] = l_run[1] * corr[1] + sum[1];
#pragma unroll
    for (int i = 0; i < 2 * NV16; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
    __syncthreads();
    const int vchunk0 = half * NV16 * 2;                         // this warp's first value chunk (8 columns each)
#pragma unroll
    for (int kk = 0; kk < (active ? BN / 16 : 0); ++kk) {
      uint32_t pf[4];
      ldmatrix_x4(pf, at(s_p, rg * 16 + (lane & 15), kk * 2 + (lane >> 4), pstride));
#pragma unroll
      for (int nb = 0; nb < 2 * NV16; nb += 2) {
        uint32_t vf[4];
        const int mi = lane >> 3;
        ldmatrix_x4_trans(vf, at(sk, kk * 16 + (mi & 1) * 8 + (lane & 7), vchunk0 + nb + (mi >> 1), stride));
        mma_bf16(o[nb], pf, vf[0], vf[1]);
        mma_bf16(o[nb + 1], pf, vf[2], vf[3]);
      }
    }
    __syncthreads();
  }
  // a pair's sum: both key halves, all four lanes of a quad
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }
  if ((lane & 3) == 0) {
    red[half * BM + r_lo] = l_run[0];
    red[half * BM + r_lo + 8] = l_run[1];
  }
  __syncthreads();
  if (split_keys > 0) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = r_lo + 8 * hh;
      if (r >= valid) continue;
      float* po = part_o + (part * BM + r) * Wv;
#pragma unroll
      for (int i = 0; i < 2 * NV16; ++i) {
        const int col = (half * NV16 * 2 + i) * 8 + 2 * (lane & 3);
        if (col < Wv) po[col] = o[i][2 * hh];
        if (col + 1 < Wv) po[col + 1] = o[i][2 * hh + 1];
      }
      if (half == 0 && (lane & 3) == 0) {
        part_ml[(part * BM + r) * 2] = m_run[hh];
        part_ml[(part * BM + r) * 2 + 1] = red[r] + red[BM + r];
      }
    }
    return;
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = r_lo + 8 * hh;
    if (r >= valid) continue;
    float inv = red[r] + red[BM + r];
    if (sink != nullptr) {      // (in the exp2 domain, like the scores)
      const float sk = sink[(pair0 + r) % H] * 1.4426950408889634f, mn = fmaxf(m_run[hh], sk);
      const float corr = exp2f(m_run[hh] - mn);
      inv = corr / (inv * corr + exp2f(sk - mn));
    } else {
      inv = 1.0f / inv;
    }
    __nv_bfloat16* orow = out + ((size_t)row0 * H + pair0 + r) * Wv;
#pragma unroll
    for (int i = 0; i < 2 * NV16; ++i) {
      const int col = (half * NV16 * 2 + i) * 8 + 2 * (lane & 3);
      if (col + 1 < Wv) *(uint32_t*)(orow + col) = pack_bf16(o[i][2 * hh] * inv, o[i][2 * hh + 1] * inv);
      else if (col < Wv) orow[col] = __float2bfloat16_rn(o[i][2 * hh] * inv);
    }
  }
}

// Adds up a tile's key ranges: out = sum_y o_y 2^(m_y - m) / sum_y l_y 2^(m_y - m), m = max_y m_y.
// One block per (tile, pair): a warp turns the ranges' (max, sum) into weights once, then every thread adds up its
// columns with independent loads. n_split <= 32.
__global__ void __launch_bounds__(256)
attn_latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ seg,
                         int n_seg, int n_split, __nv_bfloat16* __restrict__ out, int H, int Wv, const float* __restrict__ sink) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  __shared__ float w_s[32];
  __shared__ float inv_s;
  int pair0 = 0;
  const int s_idx = locate_tile(seg, n_seg, H, blockIdx.x, pair0);
  if (s_idx < 0) return;
  const int row0 = seg[4 * s_idx], valid = min(BM, seg[4 * s_idx + 1] * H - pair0);
  const int r = blockIdx.y;
  if (r >= valid) return;
  const size_t base = (size_t)blockIdx.x * n_split;
  if (threadIdx.x < 32) {
    const int y = threadIdx.x;
    const float my = y < n_split ? part_ml[((base + y) * BM + r) * 2] : -INFINITY;
    const float ly = y < n_split ? part_ml[((base + y) * BM + r) * 2 + 1] : 0.f;
    const float sk = sink != nullptr ? sink[(pair0 + r) % H] * 1.4426950408889634f : -INFINITY;
    const float m = fmaxf(warp_max(my), sk);
    const float w = ly > 0.f ? exp2f(my - m) : 0.f;      // an empty range has sum 0 (its partial output was never written)
    float l = ly * w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {                    // a prefix sum over the ranges: one fixed order of additions
      const float up = __shfl_up_sync(0xffffffffu, l, o);
      if (y >= o) l += up;
    }
    w_s[y] = w;                                            // (0 for the lanes beyond the ranges)
    if (y == 31) inv_s = 1.0f / (sink != nullptr ? l + exp2f(sk - m) : l);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < Wv; c += blockDim.x) {
    // all ranges' loads are issued before any is used (the loop has a constant bound and is unrolled); an empty range
    // (weight 0) is not read
    float v[32];
#pragma unroll
    for (int y = 0; y < 32; ++y) v[y] = (y < n_split && w_s[y] > 0.f) ? part_o[((base + y) * BM + r) * Wv + c] : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) acc = fmaf(v[y], w_s[y < n_split ? y : 0], acc);
    out[((size_t)row0 * H + pair0 + r) * Wv + c] = __float2bfloat16_rn(acc * inv_s);
  }
}

// Rows of padding (seq_row < 0) belong to no portion: their output is zero.
__global__ void zero_padding_rows_kernel(const int* __restrict__ seq_row, __nv_bfloat16* __restrict__ out, int N, int per_row) {
  fz_grid_launch_dependents();
  fz_grid_wait();
  const int n = blockIdx.x;
  if (seq_row[n] >= 0) return;
  for (int i = threadIdx.x; i < per_row; i += blockDim.x) out[(size_t)n * per_row + i] = __float2bfloat16_rn(0.f);
}

size_t smem_bytes(int W, int bn) {
  return (size_t)BM * (W + PAD) * 2 + (size_t)2 * bn * (W + PAD) * 2 + (size_t)BM * (bn + PAD) * 2 + 2 * BM * sizeof(float);
}

template <int NV16, int BN>
int launch(const void* q, const void* pool, const int* seg, int n_seg, const int* table, int mb, long long page_stride,
           int page_size, int num_pages, void* out, int blocks, int H, int W, int Wv, float scale, int window,
           float* part_o, float* part_ml, int n_split, int split_keys, const float* sink, int* err, cudaStream_t stream) {
  const size_t smem = smem_bytes(W, BN);
  auto kern = attn_latent_tc_kernel<NV16, BN>;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  fz_launch(kern, dim3(blocks, n_split), dim3(THREADS), smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, seg,
            n_seg, table, mb, page_stride, page_size, num_pages, (__nv_bfloat16*)out, H, W, Wv, scale * 1.4426950408889634f,
            window, part_o, part_ml, split_keys, err, sink);
  FZ_LAUNCH_CHECK();
  if (split_keys > 0) {
    fz_launch(attn_latent_merge_kernel, dim3(blocks, BM), dim3(256), 0, stream, (const float*)part_o, (const float*)part_ml, seg,
              n_seg, n_split, (__nv_bfloat16*)out, H, Wv, sink);
    FZ_LAUNCH_CHECK();
  }
  return FZ_OK;
}

// the value columns a warp computes, in 16s: the smallest supported count that covers Wv / 2
int nv16_for(int Wv) {
  const int want = (Wv + 31) / 32;
  for (int c : {1, 2, 3, 4, 6, 8, 12, 16})
    if (c >= want) return c;
  return 0;
}
}  // namespace

FZ_API int fz_attn_latent_tc_check(int H, int W, int Wv) {
  if (H <= 0 || W <= 0 || Wv <= 0 || Wv > W || W % 16 || Wv % 2 || W > 1024) return FZ_BAD_SHAPE;
  const int nv = nv16_for(Wv);
  if (nv == 0 || nv * 32 > W) return FZ_BAD_SHAPE;
  if (smem_bytes(W, 32) > 227 * 1024) return FZ_BAD_SHAPE;
  return FZ_OK;
}

// How a step of `blocks` tiles whose longest context is max_context is cut along the keys: the number of ranges (1: not
// cut) for a GPU of `sms` multiprocessors. Few tiles with many keys behind them (decoded tokens) would leave most of the
// GPU idle; ranges of at least 128 keys, at most 32 of them, enough for about two blocks per multiprocessor.
FZ_API int fz_attn_latent_tc_splits(int blocks, int max_context, int sms) {
  if (blocks <= 0 || blocks >= sms || max_context < 256) return 1;
  int n = (2 * sms + blocks - 1) / blocks;
  if (n > 32) n = 32;
  if (n > max_context / 128) n = max_context / 128;
  return n < 2 ? 1 : n;
}

// float32 scratch the cut needs: (outputs, then (max, sum) pairs), in floats.
FZ_API long long fz_attn_latent_tc_scratch(int blocks, int n_split, int Wv) {
  return n_split <= 1 ? 0 : (long long)blocks * n_split * BM * (Wv + 2);
}

// blocks: at least the number of 64-pair tiles of the step, sum over portions of ceil(rows * H / 64). n_split > 1: the
// keys are cut into n_split ranges of equal length (a multiple of 64) that cover max_context; scratch as above.
FZ_API int fz_attn_latent_tc(const void* q, const void* pool, const int* seq_row, const int* seg, int n_seg,
                             const int* table, int mb, long long page_stride, int page_size, int num_pages, void* out,
                             int N, int blocks, int H, int W, int Wv, float scale, int window, int n_split,
                             int max_context, float* scratch, const float* sink, int* err, cudaStream_t stream) {
  if (N <= 0) return FZ_OK;
  if (fz_attn_latent_tc_check(H, W, Wv) != FZ_OK || page_size <= 0) return FZ_BAD_SHAPE;
  if (n_split < 1 || n_split > 65535 || (n_split > 1 && scratch == nullptr)) return FZ_BAD_SHAPE;
  const int split_keys = n_split > 1 ? ((max_context + n_split - 1) / n_split + 63) / 64 * 64 : 0;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (long long)blocks * n_split * BM * Wv : nullptr;
  fz_launch(zero_padding_rows_kernel, dim3(N), dim3(128), 0, stream, seq_row, (__nv_bfloat16*)out, N, H * Wv);
  FZ_LAUNCH_CHECK();
  if (blocks <= 0 || n_seg <= 0) return FZ_OK;
  const bool wide = smem_bytes(W, 64) <= 200 * 1024;
#define FZ_GO(NV) return wide ? launch<NV, 64>(q, pool, seg, n_seg, table, mb, page_stride, page_size, num_pages, out, blocks, H, W, Wv, scale, window, part_o, part_ml, n_split, split_keys, sink, err, stream) \
                              : launch<NV, 32>(q, pool, seg, n_seg, table, mb, page_stride, page_size, num_pages, out, blocks, H, W, Wv, scale, window, part_o, part_ml, n_split, split_keys, sink, err, stream)
  switch (nv16_for(Wv)) {
    case 1: FZ_GO(1);
    case 2: FZ_GO(2);
    case 3: FZ_GO(3);
    case 4: FZ_GO(4);
    case 6: FZ_GO(6);
    case 8: FZ_GO(8);
    case 12: FZ_GO(12);
    case 16: FZ_GO(16);
  }
#undef FZ_GO
  return FZ_BAD_SHAPE;
}

#ifdef FZ_TIMELINE
FZ_TIMELINE_READER(attn_latent_tc)
#endif
