// Attention over a cached low-rank latent (one latent vector and one rotated key part per token,
// shared by all heads), on the float32 pipes.
//
// A token's cache row is [c (C numbers, RMS-normed) | r (R numbers, rotated) | zero padding to a
// multiple of 8]: pages are [page, P, row].  With the key up-projection folded into the query
// (qa[t, h] = [W_uk_h^T q_plain | q_rotated], done by the caller with two products), a head's score
// against key j is qa[t, h] . row_j, and its output in latent space is sum_j p_j c_j: every head
// attends over the same rows, and the values are the first C numbers of the keys.
//
//   flint_latent_prepare    sums the partial sums of the q (and latent) projection, rotates the
//                           rotated parts (neighbouring dims 2i, 2i+1 or halves i, i+n/2), norms the
//                           latent and writes the cache row; q_plain and the rotated q part go out
//                           in the activation type
//   flint_latent_attention  one warp per (row, chunk of 4 heads, split of the key range): a lane owns
//                           a key in the score phase and output dims lane, lane+32, ... in the value
//                           phase; online softmax in float32; splits are merged in a fixed order
//
// The reference has no such mixer (its attention is grouped-query over cached keys and values:
// crates/thuban_kernel/wgsl/attn.wgsl); these kernels have no counterpart there.
#include "attention_kernels.cuh"

using namespace flint;
using flint_attn::load8;

namespace {
constexpr int GC = 4;           // heads per warp
constexpr int WARPS = 4;
constexpr int MAX_DPL = 16;     // output dims per lane: latent size <= 512

template <typename TQ, typename TC>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, int n_partials, long long partial_stride, int W,
                      const int* __restrict__ pos, const int* __restrict__ slot,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims, int interleaved,
                      const float* __restrict__ norm_w, float eps, TQ* __restrict__ q_plain, TQ* __restrict__ qa,
                      TC* __restrict__ k_cache, const int* __restrict__ block_table, int max_pages, int page_size,
                      int H, int D, int R, int C, int row_w, int write_kv, int* __restrict__ status) {
  extern __shared__ float sm[];         // C floats of the latent before its norm
  __shared__ float red[32];
  pdl_launch();
  const int t = blockIdx.x;
  const int p = pos[t];
  long long cache_row = -1;
  bool missing = false;
  if (write_kv) {
    const int page = block_table[(size_t)slot[t] * max_pages + p / page_size];
    if (page >= 0) cache_row = (long long)page * page_size + p % page_size;
    else missing = true;
  }
  pdl_wait();
  if (missing && threadIdx.x == 0) atomicExch(status, 1);
  const float* row = proj + (size_t)t * W;
  auto total = [&](int col) {
    float s = 0.f;
    for (int z = 0; z < n_partials; ++z) s += row[(size_t)z * partial_stride + col];
    return s;
  };
  const int half = rot_dims / 2, DR = D + R, Dk = C + R;
  const int units = half + (R - rot_dims);        // rotating pairs, then the dims that pass unchanged
  // the pair of unit u (< half) and the rotation of (a, b) by the angle of pair u at position p
  auto dims_of = [&](int u, int& d0, int& d1) {
    if (interleaved) { d0 = 2 * u; d1 = 2 * u + 1; }
    else { d0 = u; d1 = u + half; }
  };
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
    const int h = i / D, d = i - h * D;
    q_plain[((size_t)t * H + h) * D + d] = from_f32<TQ>(total(h * DR + d));
  }
  for (int i = threadIdx.x; i < H * units; i += blockDim.x) {
    const int h = i / units, u = i - h * units;
    const int src = h * DR + D;
    TQ* dst = qa + ((size_t)t * H + h) * Dk + C;
    if (u < half) {
      int d0, d1;
      dims_of(u, d0, d1);
      const float a = total(src + d0), b = total(src + d1);
      const float c = cos_t[(size_t)p * half + u], s = sin_t[(size_t)p * half + u];
      dst[d0] = from_f32<TQ>(a * c - b * s);
      dst[d1] = from_f32<TQ>(b * c + a * s);
    } else {
      const int d = rot_dims + (u - half);
      dst[d] = from_f32<TQ>(total(src + d));
    }
  }
  if (!write_kv) return;
  const int base = H * DR;
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const float v = total(base + i);
    sm[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)C + eps);
  if (cache_row < 0) return;
  TC* dst = k_cache + cache_row * row_w;
  for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = from_f32<TC>(sm[i] * inv * norm_w[i]);
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    if (u < half) {
      int d0, d1;
      dims_of(u, d0, d1);
      const float a = total(base + C + d0), b = total(base + C + d1);
      const float c = cos_t[(size_t)p * half + u], s = sin_t[(size_t)p * half + u];
      dst[C + d0] = from_f32<TC>(a * c - b * s);
      dst[C + d1] = from_f32<TC>(b * c + a * s);
    } else {
      const int d = rot_dims + (u - half);
      dst[C + d] = from_f32<TC>(total(base + C + d));
    }
  }
  for (int i = Dk + threadIdx.x; i < row_w; i += blockDim.x) dst[i] = from_f32<TC>(0.f);
}

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_kernel(const TQ* __restrict__ qa, const TC* __restrict__ k_cache, const int* __restrict__ block_table,
                        int max_pages, int page_size, const int* __restrict__ pos, const int* __restrict__ slot,
                        TO* __restrict__ out, float* __restrict__ scratch, int T, int H, int C, int Dk, int row_w,
                        int window, float scale, int split_keys, int n_splits, int g_chunks,
                        const int* __restrict__ row_list) {
  extern __shared__ float smem[];   // per warp: GC * row_w floats of q
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  const long long n_items = (long long)T * g_chunks * n_splits;
  if (item >= n_items) return;
  const int split = (int)(item % n_splits);
  long long rest = item / n_splits;
  const int gchunk = (int)(rest % g_chunks);
  const int ti = (int)(rest / g_chunks);
  const int t = row_list ? row_list[ti] : ti;
  const int h0 = gchunk * GC;
  const int ng = min(GC, H - h0);
  const int p = pos[t];
  const int lo_row = window > 0 ? max(0, p + 1 - window) : 0;
  const int lo = lo_row + split * split_keys;
  const int hi = min(p + 1, lo + split_keys);
  const int* bt = block_table + (size_t)slot[t] * max_pages;

  float* qs = smem + (size_t)warp * GC * row_w;
  for (int i = lane; i < GC * row_w; i += 32) {
    const int g = i / row_w, d = i - g * row_w;
    qs[i] = (g < ng && d < Dk) ? to_f32(qa[((size_t)t * H + h0 + g) * Dk + d]) * scale : 0.f;
  }
  __syncwarp();

  const int dpl = (C + 31) / 32;
  float m[GC], l[GC], acc[GC][MAX_DPL];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) acc[g][i] = 0.f;
  }
  for (int j0 = lo; j0 < hi; j0 += 32) {
    const int j = j0 + lane;
    long long row = -1;
    if (j < hi) {
      const int page = bt[j / page_size];
      if (page >= 0) row = (long long)page * page_size + (j % page_size);
    }
    float s[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) s[g] = 0.f;
    if (row >= 0) {
      const TC* kr = k_cache + row * row_w;
      for (int d = 0; d < row_w; d += 8) {     // the row width is a multiple of 8
        float kf[8];
        load8<TC>(kr + d, kf);
#pragma unroll
        for (int g = 0; g < GC; ++g)
          if (g < ng) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s[g] = fmaf(qs[g * row_w + d + e], kf[e], s[g]);
          }
      }
    }
    float pr[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      const float sg = row >= 0 ? s[g] : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(sg));
      const bool any = m_new > -INFINITY;
      const float alpha = any ? expf(m[g] - m_new) : 1.f;
      pr[g] = (any && row >= 0) ? expf(sg - m_new) : 0.f;
      l[g] = l[g] * alpha + warp_sum(pr[g]);
      m[g] = m_new;
#pragma unroll
      for (int i = 0; i < MAX_DPL; ++i) acc[g][i] *= alpha;
    }
    const int nk = min(32, hi - j0);
    for (int jj = 0; jj < nk; ++jj) {
      const long long vrow = __shfl_sync(0xffffffffu, row, jj);
      float pj[GC];
#pragma unroll
      for (int g = 0; g < GC; ++g) pj[g] = __shfl_sync(0xffffffffu, pr[g], jj);
      if (vrow < 0) continue;
      const TC* vr = k_cache + vrow * row_w;
#pragma unroll
      for (int i = 0; i < MAX_DPL; ++i) {
        const int d = lane + 32 * i;
        if (i < dpl && d < C) {
          const float vv = to_f32(vr[d]);
#pragma unroll
          for (int g = 0; g < GC; ++g) acc[g][i] = fmaf(pj[g], vv, acc[g][i]);
        }
      }
    }
  }
  if (n_splits == 1) {
#pragma unroll
    for (int g = 0; g < GC; ++g)
      if (g < ng) {
        const float inv = l[g] > 0.f ? 1.0f / l[g] : 0.f;
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) {
          const int d = lane + 32 * i;
          if (i < dpl && d < C) out[((size_t)t * H + h0 + g) * C + d] = from_f32<TO>(acc[g][i] * inv);
        }
      }
  } else {
    // scratch [T, H, n_splits, C + 2]: unnormalised output, then max, then sum
#pragma unroll
    for (int g = 0; g < GC; ++g)
      if (g < ng) {
        float* dst = scratch + (((size_t)ti * H + h0 + g) * n_splits + split) * (C + 2);
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) {
          const int d = lane + 32 * i;
          if (i < dpl && d < C) dst[d] = acc[g][i];
        }
        if (lane == 0) {
          dst[C] = m[g];
          dst[C + 1] = l[g];
        }
      }
  }
}
// ---------------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16 in, float32 scores, sums and outputs).
//
// A block of 8 warps takes up to 32 query rows, a row being one (token, head) pair: `nt` consecutive tokens
// of the batch by `nh` heads.  All rows of a request attend over the same cached rows, so the block
// streams tiles of 64 keys through shared memory once for all of them (tokens of different requests in a
// block are worked one run after the other).  Per tile: warp (wm, wk) computes the scores of query rows
// [16 wm, +16) against keys [16 wk, +16) with mma.sync m16n8k16 (Q and K through ldmatrix), the four
// warps of a row tile agree on the new maximum and sum through shared memory, the probabilities go to
// shared memory as bfloat16, and the warp then adds P V for ITS quarter of the latent dims (V is the start
// of the key rows already in shared memory, through ldmatrix.trans): the output accumulator of 16 rows by
// up to 128 dims stays in registers.  Tiles arrive by asynchronous copies into two buffers: the next tile is on
// its way while this one is worked.  Causal and window masks are per row.  With n_splits > 1 the key
// range of a run is cut and the pieces are merged by attention_combine_kernel.
constexpr int TM = 32;        // query rows per block
constexpr int KT = 64;        // keys per tile
constexpr int TC_THREADS = 256;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ float ex2(float x) {          // 2^x; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NTW>            // blocks of 8 latent dims per warp in the value phase: latent size <= 32 NTW
__global__ void __launch_bounds__(TC_THREADS)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ qa, const __nv_bfloat16* __restrict__ k_cache,
                            const int* __restrict__ block_table, int max_pages, int page_size,
                            const int* __restrict__ pos, const int* __restrict__ slot, __nv_bfloat16* __restrict__ out,
                            float* __restrict__ scratch, int T, int H, int C, int Dk, int row_w, int Dkp, int window,
                            float scale, int nt, int nh, int split_keys, int n_splits) {
  using flint_attn::ldsm4;
  using flint_attn::ldsm4t;
  using flint_attn::mma16816;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int QS = Dkp + 8;                                        // row stride of Qs and Ks (elements): odd in 16-byte units
  constexpr int PS = KT + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Kb = Qs + (size_t)TM * QS;                      // two buffers of KT rows, filled by asynchronous copies
  const size_t kbuf = (size_t)KT * QS;
  __nv_bfloat16* Ps = Kb + 2 * kbuf + 512;                       // slack: the value phase may read columns past a row's end
  float* redm = reinterpret_cast<float*>(Ps + TM * PS);          // [TM][4]
  float* reds = redm + TM * 4;                                   // [TM][4]
  int* kval = reinterpret_cast<int*>(reds + TM * 4);             // [2][KT]: whether each key of a buffered tile has a page
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 2, wk = warp & 3;
  // the last tokens first: in a prompt's portion they see the most keys, and the short blocks fill in behind them
  const int t_first = (gridDim.x - 1 - blockIdx.x) * nt, h0 = blockIdx.y * nh, split = blockIdx.z;
  const int ntok = min(nt, T - t_first), nhh = min(nh, H - h0);
  const int r_lo = wm * 16 + (lane >> 2), r_hi = r_lo + 8;       // the two query rows of this lane's fragments
  const float scale2 = scale * 1.4426950408889634f;              // scores are kept in units of log 2
  const int cpr = Dkp / 8;                                       // 16-byte units per staged row
  const int row_units = row_w / 8;                               // of which the cached row fills so many
  pdl_launch();
  // a staged row may be one unit wider than the cached row: that unit stays zero in both buffers
  if (row_units < cpr)
    for (int r = tid; r < 2 * KT; r += TC_THREADS)
      *reinterpret_cast<uint4*>(Kb + (size_t)r * QS + row_units * 8) = make_uint4(0u, 0u, 0u, 0u);
  pdl_wait();

  int ta = 0;
  while (ta < ntok) {
    const int s = slot[t_first + ta];
    int tb = ta + 1;
    while (tb < ntok && slot[t_first + tb] == s && pos[t_first + tb] == pos[t_first + tb - 1] + 1) ++tb;
    const int n_rows = (tb - ta) * nhh;
    const int p_a = pos[t_first + ta], p_b = p_a + (tb - ta) - 1;
    const int lo_run = window > 0 ? max(0, p_a + 1 - window) : 0;
    const int lo = lo_run + split * split_keys;
    const int hi = min(p_b + 1, lo + split_keys);
    const int* bt = block_table + (size_t)s * max_pages;
    // the run's query rows, zero beyond the row's width and beyond the run
    if ((Dk & 7) == 0) {
      for (int c = tid; c < TM * cpr; c += TC_THREADS) {
        const int r = c / cpr, cu = c - r * cpr;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_rows && cu * 8 < Dk) {
          const int tok = t_first + ta + r / nhh, h = h0 + r % nhh;
          v = *reinterpret_cast<const uint4*>(qa + ((size_t)tok * H + h) * Dk + cu * 8);
        }
        *reinterpret_cast<uint4*>(Qs + (size_t)r * QS + cu * 8) = v;
      }
    } else {
      for (int e = tid; e < TM * Dkp; e += TC_THREADS) {
        const int r = e / Dkp, d = e - r * Dkp;
        __nv_bfloat16 v = __float2bfloat16_rn(0.f);
        if (r < n_rows && d < Dk) {
          const int tok = t_first + ta + r / nhh, h = h0 + r % nhh;
          v = qa[((size_t)tok * H + h) * Dk + d];
        }
        Qs[(size_t)r * QS + d] = v;
      }
    }
    // a tile's rows are fetched by asynchronous 16-byte copies (zeros where there is no key): thread t brings
    // every fourth unit of key t / 4, so it looks the key's page up once
    auto row_of_key = [&](int j0) {            // the cache row of this thread's key of the tile at j0, or -1
      const int j = j0 + (tid >> 2);
      if (j >= hi) return -1ll;
      const int page = bt[j / page_size];
      return page >= 0 ? (long long)page * page_size + (j % page_size) : -1ll;
    };
    long long next_row = lo < hi ? row_of_key(lo) : -1ll;    // looked up a tile ahead of its use
    auto fetch = [&](int j0, int buf) {
      const int jj = tid >> 2;
      const long long row = next_row;
      next_row = row_of_key(j0 + KT);
      if ((tid & 3) == 0) kval[buf * KT + jj] = row >= 0;
      const __nv_bfloat16* src = k_cache + (row >= 0 ? row * row_w : 0) + (tid & 3) * 8;
      uint32_t dst = smem_addr(Kb + buf * kbuf + (size_t)jj * QS) + (tid & 3) * 16;
      const int size = row >= 0 ? 16 : 0;                        // no key: the units are filled with zeros
      for (int cu = tid & 3; cu < row_units; cu += 4, src += 32, dst += 64)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(size) : "memory");
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int p_lo = p_a + r_lo / nhh, p_hi = p_a + r_hi / nhh;   // positions of this lane's rows (if they are in the run)
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[NTW][4];
#pragma unroll
    for (int i = 0; i < NTW; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    if (lo < hi) fetch(lo, 0);
    int buf = 0;
    for (int j0 = lo; j0 < hi; j0 += KT, buf ^= 1) {
      if (j0 + KT < hi) {
        fetch(j0 + KT, buf ^ 1);                                   // that buffer's last readers passed the barrier below
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();
      const __nv_bfloat16* Ks = Kb + buf * kbuf;
      const int* kv_ok = kval + buf * KT;
      // ---- scores of 16 rows x 16 keys
      float sc[2][4], sd[2][4];       // even and odd steps of the dims add into accumulators of their own: two chains
#pragma unroll
      for (int n = 0; n < 2; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f; sd[n][0] = sd[n][1] = sd[n][2] = sd[n][3] = 0.f; }
      {
        const uint32_t qaddr = smem_addr(Qs + (size_t)(wm * 16 + (lane & 15)) * QS + (lane >> 4) * 8);
        const uint32_t kaddr = smem_addr(Ks + (size_t)(wk * 16 + ((lane >> 4) << 3) + (lane & 7)) * QS + ((lane >> 3) & 1) * 8);
        int kk = 0;
#pragma unroll 2
        for (; kk + 32 <= Dkp; kk += 32) {
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3, c0, c1, c2, c3, d0, d1, d2, d3;
          ldsm4(qaddr + kk * 2, a0, a1, a2, a3);
          ldsm4(kaddr + kk * 2, b0, b1, b2, b3);
          ldsm4(qaddr + kk * 2 + 32, c0, c1, c2, c3);
          ldsm4(kaddr + kk * 2 + 32, d0, d1, d2, d3);
          mma16816(sc[0], a0, a1, a2, a3, b0, b1);
          mma16816(sc[1], a0, a1, a2, a3, b2, b3);
          mma16816(sd[0], c0, c1, c2, c3, d0, d1);
          mma16816(sd[1], c0, c1, c2, c3, d2, d3);
        }
        if (kk < Dkp) {
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          ldsm4(qaddr + kk * 2, a0, a1, a2, a3);
          ldsm4(kaddr + kk * 2, b0, b1, b2, b3);
          mma16816(sc[0], a0, a1, a2, a3, b0, b1);
          mma16816(sc[1], a0, a1, a2, a3, b2, b3);
        }
#pragma unroll
        for (int n = 0; n < 2; ++n) { sc[n][0] += sd[n][0]; sc[n][1] += sd[n][1]; sc[n][2] += sd[n][2]; sc[n][3] += sd[n][3]; }
      }
      // scores in units of log 2 (the scale carries log2 e), so that the exponentials are single instructions; a tile
      // that every row of the run sees whole needs no masks
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
      const bool whole = j0 + KT <= hi && j0 + KT - 1 <= p_a && (window <= 0 || j0 > p_b - window) && n_rows == TM;
      if (whole) {
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          sc[n][0] *= scale2; sc[n][1] *= scale2; sc[n][2] *= scale2; sc[n][3] *= scale2;
          mx_lo = fmaxf(mx_lo, fmaxf(sc[n][0], sc[n][1]));
          mx_hi = fmaxf(mx_hi, fmaxf(sc[n][2], sc[n][3]));
        }
      } else {
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int j = j0 + wk * 16 + n * 8 + 2 * (lane & 3) + (i & 1);
            const int r = i < 2 ? r_lo : r_hi, p = i < 2 ? p_lo : p_hi;
            const bool seen = r < n_rows && j < hi && j <= p && (window <= 0 || j > p - window) && kv_ok[j - j0];
            sc[n][i] = seen ? sc[n][i] * scale2 : -INFINITY;
            if (i < 2) mx_lo = fmaxf(mx_lo, sc[n][i]); else mx_hi = fmaxf(mx_hi, sc[n][i]);
          }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      if ((lane & 3) == 0) { redm[r_lo * 4 + wk] = mx_lo; redm[r_hi * 4 + wk] = mx_hi; }
      __syncthreads();
      float mn_lo = m_lo, mn_hi = m_hi;
#pragma unroll
      for (int w = 0; w < 4; ++w) { mn_lo = fmaxf(mn_lo, redm[r_lo * 4 + w]); mn_hi = fmaxf(mn_hi, redm[r_hi * 4 + w]); }
      // a row that has seen no key yet keeps m = -inf; its exponentials are taken against 0 and come out 0
      const float ref_lo = mn_lo > -INFINITY ? mn_lo : 0.f, ref_hi = mn_hi > -INFINITY ? mn_hi : 0.f;
      const float al_lo = mn_lo == m_lo ? 1.f : ex2(m_lo - ref_lo);
      const float al_hi = mn_hi == m_hi ? 1.f : ex2(m_hi - ref_hi);
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const float p0 = ex2(sc[n][0] - ref_lo), p1 = ex2(sc[n][1] - ref_lo);
        const float p2 = ex2(sc[n][2] - ref_hi), p3 = ex2(sc[n][3] - ref_hi);
        sum_lo += p0 + p1;
        sum_hi += p2 + p3;
        const int col = wk * 16 + n * 8 + 2 * (lane & 3);
        *reinterpret_cast<__nv_bfloat162*>(Ps + r_lo * PS + col) = __floats2bfloat162_rn(p0, p1);
        *reinterpret_cast<__nv_bfloat162*>(Ps + r_hi * PS + col) = __floats2bfloat162_rn(p2, p3);
      }
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
      sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
      sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
      if ((lane & 3) == 0) { reds[r_lo * 4 + wk] = sum_lo; reds[r_hi * 4 + wk] = sum_hi; }
      __syncthreads();
      l_lo = l_lo * al_lo + (reds[r_lo * 4] + reds[r_lo * 4 + 1] + reds[r_lo * 4 + 2] + reds[r_lo * 4 + 3]);
      l_hi = l_hi * al_hi + (reds[r_hi * 4] + reds[r_hi * 4 + 1] + reds[r_hi * 4 + 2] + reds[r_hi * 4 + 3]);
      m_lo = mn_lo;
      m_hi = mn_hi;
      // ---- O += P V for this warp's dims [32 NTW wk / 4 ...): 16 rows x 8 NTW dims
      if (__any_sync(0xffffffffu, al_lo != 1.f || al_hi != 1.f)) {     // a maximum moved: rescale what was added so far
#pragma unroll
        for (int i = 0; i < NTW; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
      }
      {
        const uint32_t paddr = smem_addr(Ps + (wm * 16 + (lane & 15)) * PS + (lane >> 4) * 8);
        const uint32_t vaddr = smem_addr(Ks + (size_t)((((lane >> 3) & 1) << 3) + (lane & 7)) * QS + (lane >> 4) * 8);
#pragma unroll
        for (int ks = 0; ks < KT / 16; ++ks) {
          uint32_t a0, a1, a2, a3;
          ldsm4(paddr + ks * 32, a0, a1, a2, a3);
#pragma unroll
          for (int nb = 0; nb < NTW; nb += 2) {
            const int col = (wk * NTW + nb) * 8;
            if (col < C) {
              uint32_t b0, b1, b2, b3;
              ldsm4t(vaddr + (uint32_t)(((size_t)ks * 16 * QS + col) * 2), b0, b1, b2, b3);
              mma16816(o[nb], a0, a1, a2, a3, b0, b1);
              mma16816(o[nb + 1], a0, a1, a2, a3, b2, b3);
            }
          }
        }
      }
      __syncthreads();
    }
    // ---- this run's rows go out
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? r_hi : r_lo;
      if (r < n_rows) {
        const int tok = t_first + ta + r / nhh, h = h0 + r % nhh;
        const float m = half ? m_hi : m_lo, l = half ? l_hi : l_lo;
        if (n_splits == 1) {
          const float inv = l > 0.f ? 1.0f / l : 0.f;
          __nv_bfloat16* dst = out + ((size_t)tok * H + h) * C;
#pragma unroll
          for (int nb = 0; nb < NTW; ++nb) {
            const int col = (wk * NTW + nb) * 8 + 2 * (lane & 3);
            if (col < C) dst[col] = __float2bfloat16_rn(o[nb][2 * half] * inv);
            if (col + 1 < C) dst[col + 1] = __float2bfloat16_rn(o[nb][2 * half + 1] * inv);
          }
        } else {
          float* dst = scratch + (((size_t)tok * H + h) * n_splits + split) * (C + 2);
#pragma unroll
          for (int nb = 0; nb < NTW; ++nb) {
            const int col = (wk * NTW + nb) * 8 + 2 * (lane & 3);
            if (col < C) dst[col] = o[nb][2 * half];
            if (col + 1 < C) dst[col + 1] = o[nb][2 * half + 1];
          }
          if (wk == 0 && (lane & 3) == 0) { dst[C] = m * 0.6931471805599453f; dst[C + 1] = l; }   // the merge works in natural logarithms
        }
      }
    }
    __syncthreads();
    ta = tb;
  }
}
// ---------------------------------------------------------------------------------------------
// A small product per head, all heads in one launch: out[t, h, :] = W[h] x[t, h, :] (bfloat16 in and out,
// float32 sums).  x and out may be views into wider rows (strides in elements).  Block (64 tokens, 64 outputs,
// head): four warps of 16 tokens each, operands staged in shared memory 64 columns at a time, the next stage on
// its way while this one is multiplied.
constexpr int HP_M = 64, HP_N = 64, HP_K = 64, HP_S = HP_K + 8;

__global__ void __launch_bounds__(128)
head_products_kernel(const __nv_bfloat16* __restrict__ x, long long sx_t, long long sx_h,
                     const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long so_t,
                     long long so_h, int T, int N, int K) {
  using flint_attn::ldsm4;
  using flint_attn::mma16816;
  __shared__ __align__(16) __nv_bfloat16 As[2][HP_M * HP_S];      // two stages, filled by asynchronous copies
  __shared__ __align__(16) __nv_bfloat16 Bs[2][HP_N * HP_S];
  pdl_launch();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = blockIdx.x * HP_M, n0 = blockIdx.y * HP_N, h = blockIdx.z;
  const __nv_bfloat16* xh = x + (size_t)h * sx_h;
  const __nv_bfloat16* wh = w + (size_t)h * N * K;
  float acc[HP_N / 8][4];
#pragma unroll
  for (int i = 0; i < HP_N / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  auto fetch = [&](int k0, int st) {            // 16-byte units of both operands; zeros beyond the edges
    for (int c = tid; c < (HP_M + HP_N) * (HP_K / 8); c += 128) {
      const int r = c / (HP_K / 8), cu = c % (HP_K / 8), k = k0 + cu * 8;
      const __nv_bfloat16* src;
      uint32_t dst;
      bool live;
      if (r < HP_M) {
        live = t0 + r < T && k < K;
        src = xh + (size_t)(t0 + r) * sx_t + k;
        dst = smem_addr(As[st] + r * HP_S + cu * 8);
      } else {
        const int n = r - HP_M;
        live = n0 + n < N && k < K;
        src = wh + (size_t)(n0 + n) * K + k;
        dst = smem_addr(Bs[st] + n * HP_S + cu * 8);
      }
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(live ? src : x), "r"(live ? 16 : 0) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  pdl_wait();
  fetch(0, 0);
  int st = 0;
  for (int k0 = 0; k0 < K; k0 += HP_K, st ^= 1) {
    if (k0 + HP_K < K) {
      fetch(k0 + HP_K, st ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HP_K; kk += 16) {
      uint32_t a0, a1, a2, a3;
      ldsm4(smem_addr(As[st] + (warp * 16 + (lane & 15)) * HP_S + kk + (lane >> 4) * 8), a0, a1, a2, a3);
#pragma unroll
      for (int nb = 0; nb < HP_N / 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        ldsm4(smem_addr(Bs[st] + (nb * 8 + ((lane >> 4) << 3) + (lane & 7)) * HP_S + kk + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
        mma16816(acc[nb], a0, a1, a2, a3, b0, b1);
        mma16816(acc[nb + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int t = t0 + warp * 16 + (lane >> 2) + 8 * half;
    if (t >= T) continue;
    __nv_bfloat16* dst = out + (size_t)t * so_t + (size_t)h * so_h;
#pragma unroll
    for (int nb = 0; nb < HP_N / 8; ++nb) {
      const int n = n0 + nb * 8 + 2 * (lane & 3);
      if (n < N) dst[n] = __float2bfloat16_rn(acc[nb][2 * half]);
      if (n + 1 < N) dst[n + 1] = __float2bfloat16_rn(acc[nb][2 * half + 1]);
    }
  }
}

// The same for a handful of tokens (decoded tokens): a warp per output (h, n) reads its weight row once, all loads in
// flight, and forms the dot products with every token's row (staged in shared memory as float32).
constexpr int HPS_T = 16;        // tokens at most
__global__ void __launch_bounds__(256)
head_products_small_kernel(const __nv_bfloat16* __restrict__ x, long long sx_t, long long sx_h,
                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long so_t,
                           long long so_h, int T, int N, int K) {
  extern __shared__ float xs[];                  // [T][K]
  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, n = blockIdx.x * 8 + warp;
  // the weight row is no kernel's output: its first units are asked for before the wait
  const __nv_bfloat16* wrow = w + ((size_t)h * N + min(n, N - 1)) * K;
  uint4 first = make_uint4(0u, 0u, 0u, 0u);
  if (lane * 8 < K) first = *reinterpret_cast<const uint4*>(wrow + lane * 8);
  pdl_wait();
  for (int i = threadIdx.x; i < T * (K / 8); i += 256) {
    const int t = i / (K / 8), cu = i - t * (K / 8);
    float f[8];
    load8<__nv_bfloat16>(x + (size_t)t * sx_t + (size_t)h * sx_h + cu * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) xs[t * K + cu * 8 + e] = f[e];
  }
  __syncthreads();
  if (n >= N) return;
  float acc[HPS_T];
#pragma unroll
  for (int t = 0; t < HPS_T; ++t) acc[t] = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 raw = k == lane * 8 ? first : *reinterpret_cast<const uint4*>(wrow + k);
    float wf[8];
    const uint32_t ww[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wf[2 * i] = __uint_as_float(ww[i] << 16);
      wf[2 * i + 1] = __uint_as_float(ww[i] & 0xffff0000u);
    }
#pragma unroll
    for (int t = 0; t < HPS_T; ++t)
      if (t < T) {
        const float4 x0 = *reinterpret_cast<const float4*>(xs + t * K + k), x1 = *reinterpret_cast<const float4*>(xs + t * K + k + 4);
        acc[t] += wf[0] * x0.x + wf[1] * x0.y + wf[2] * x0.z + wf[3] * x0.w + wf[4] * x1.x + wf[5] * x1.y + wf[6] * x1.z + wf[7] * x1.w;
      }
  }
#pragma unroll
  for (int t = 0; t < HPS_T; ++t)
    if (t < T) {
      const float v = warp_sum(acc[t]);
      if (lane == 0) out[(size_t)t * so_t + (size_t)h * so_h + n] = __float2bfloat16_rn(v);
    }
}
}  // namespace

// proj [S, T, W] float32 partial sums of [q | latent] (W = H (D + R) + (write_kv ? C + R : 0)); q_plain
// [T, H, D] and qa [T, H, C + R] (only its last R numbers per head are written) in q_dtype; the cache row
// of each token (row_w numbers, a multiple of 8, at least C + R) in cache_dtype.
extern "C" int flint_latent_prepare(const float* proj, int n_partials, long long partial_stride, const int* pos,
                                    const int* slot, const float* cos_t, const float* sin_t, int rot_dims,
                                    int interleaved, const float* norm_w, float eps, void* q_plain, void* qa,
                                    int q_dtype, void* k_cache, int cache_dtype, const int* block_table,
                                    int max_pages, int page_size, int T, int H, int D, int R, int C, int row_w,
                                    int write_kv, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_partials < 1) return fail("latent_prepare: needs at least one partial");
  if (H < 1 || D < 0 || R < 0 || C < 1) return fail("latent_prepare: bad sizes H=%d D=%d R=%d C=%d", H, D, R, C);
  if (rot_dims < 0 || rot_dims > R || (rot_dims & 1)) return fail("latent_prepare: %d rotating dims do not fit %d", rot_dims, R);
  if (write_kv && (row_w < C + R || (row_w & 7))) return fail("latent_prepare: cache rows of %d numbers do not hold %d", row_w, C + R);
  if (write_kv && (!k_cache || !norm_w || page_size <= 0)) return fail("latent_prepare: no cache to write to");
  const int W = H * (D + R) + (write_kv ? C + R : 0);
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 48 * 1024) return fail("latent_prepare: latent size %d is too large", C);
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC,
      (launch_pdl(latent_prepare_kernel<TQ, TC>, dim3(T), dim3(256), smem, stream, proj, n_partials, partial_stride, W,
                  pos, slot, cos_t, sin_t, rot_dims, interleaved, norm_w, eps, (TQ*)q_plain, (TQ*)qa, (TC*)k_cache,
                  block_table, max_pages, page_size, H, D, R, C, row_w, write_kv, status))));
  return check_launch("latent_prepare");
}

// qa [T, H, Dk] -> out [T, H, C] (both q_dtype); scratch holds T*H*n_splits*(C+2) floats when n_splits > 1.
extern "C" int flint_latent_attention(const void* qa, int q_dtype, const void* k_cache, int cache_dtype,
                                      const int* block_table, int max_pages, int page_size, const int* pos,
                                      const int* slot, void* out, int T, int H, int C, int Dk, int row_w, int window,
                                      float scale, int split_keys, int n_splits, float* scratch,
                                      const int* row_list, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C < 1 || C > 32 * MAX_DPL) return fail("latent_attention: latent size %d (supported: 1..%d)", C, 32 * MAX_DPL);
  if (Dk < C || row_w < Dk || (row_w & 7)) return fail("latent_attention: bad row sizes C=%d Dk=%d row=%d", C, Dk, row_w);
  if (n_splits < 1 || split_keys < 1) return fail("latent_attention: bad split (%d keys, %d splits)", split_keys, n_splits);
  if (n_splits > 1 && !scratch) return fail("latent_attention: splits need scratch memory");
  const int g_chunks = (H + GC - 1) / GC;
  const long long items = (long long)T * g_chunks * n_splits;
  const long long blocks = (items + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return fail("latent_attention: too many work items");
  const size_t smem = (size_t)WARPS * GC * row_w * sizeof(float);
  if (smem > 200 * 1024) return fail("latent_attention: rows of %d numbers are too wide", row_w);
#define LAUNCH(TQ, TC)                                                                                          \
  do {                                                                                                          \
    if (smem > 48 * 1024)                                                                                       \
      cudaFuncSetAttribute(latent_attention_kernel<TQ, TC, TQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                           200 * 1024);                                                                         \
    latent_attention_kernel<TQ, TC, TQ><<<(unsigned)blocks, WARPS * 32, smem, stream>>>(                        \
        (const TQ*)qa, (const TC*)k_cache, block_table, max_pages, page_size, pos, slot, (TQ*)out, scratch, T,  \
        H, C, Dk, row_w, window, scale, split_keys, n_splits, g_chunks, row_list);                              \
  } while (0)
  FLINT_DISPATCH_DTYPE(q_dtype, TQ, FLINT_DISPATCH_DTYPE(cache_dtype, TC, LAUNCH(TQ, TC)));
#undef LAUNCH
  int rc = check_launch("latent_attention");
  if (rc || n_splits == 1) return rc;
  const int threads = C >= 128 ? 128 : 64;
  FLINT_DISPATCH_DTYPE(q_dtype, TO,
      (flint_attn::attention_combine_kernel<TO><<<(unsigned)((long long)T * H), threads, 0, stream>>>(
          scratch, (TO*)out, C, n_splits, H, row_list)));
  return check_launch("latent_attention (merge)");
}

// The same on the tensor cores: bfloat16 qa, cache and out.  Blocks take `nt` consecutive tokens of the batch by
// `nh` heads (nt * nh <= 32).
extern "C" int flint_latent_attention_mma(const void* qa, const void* k_cache, const int* block_table, int max_pages,
                                          int page_size, const int* pos, const int* slot, void* out, int T, int H, int C,
                                          int Dk, int row_w, int window, float scale, int nt, int nh, int split_keys,
                                          int n_splits, float* scratch, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C < 1 || C > 512) return fail("latent_attention: latent size %d (supported: 1..512)", C);
  if (Dk < C || row_w < Dk || (row_w & 7)) return fail("latent_attention: bad row sizes C=%d Dk=%d row=%d", C, Dk, row_w);
  if (nt < 1 || nh < 1 || nt * nh > TM) return fail("latent_attention: %d tokens by %d heads do not fit a block of %d rows", nt, nh, TM);
  if (n_splits < 1 || split_keys < 1) return fail("latent_attention: bad split (%d keys, %d splits)", split_keys, n_splits);
  if (n_splits > 1 && !scratch) return fail("latent_attention: splits need scratch memory");
  if (((uintptr_t)k_cache & 15) != 0) return fail("latent_attention: the cache must be 16-byte aligned");
  const int Dkp = (row_w + 15) / 16 * 16;
  const int QS = Dkp + 8;
  const size_t smem = ((size_t)TM * QS + 2 * (size_t)KT * QS + 512 + (size_t)TM * (KT + 8)) * sizeof(__nv_bfloat16) +
                      (size_t)TM * 8 * sizeof(float) + 2 * KT * sizeof(int);
  if (smem > 220 * 1024) return fail("latent_attention: rows of %d numbers are too wide", row_w);
  dim3 grid((T + nt - 1) / nt, (H + nh - 1) / nh, n_splits);
  if (grid.y > 65535 || grid.z > 65535) return fail("latent_attention: too many head chunks or splits");
#define LAUNCH(N)                                                                                                     \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(latent_attention_mma_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);  \
    launch_pdl(latent_attention_mma_kernel<N>, grid, dim3(TC_THREADS), smem, stream,                                  \
               (const __nv_bfloat16*)qa, (const __nv_bfloat16*)k_cache, block_table, max_pages, page_size, pos, slot, \
               (__nv_bfloat16*)out, scratch, T, H, C, Dk, row_w, Dkp, window, scale, nt, nh, split_keys, n_splits);   \
  } while (0)
  if (C <= 64) LAUNCH(2);
  else if (C <= 128) LAUNCH(4);
  else if (C <= 256) LAUNCH(8);
  else LAUNCH(16);
#undef LAUNCH
  int rc = check_launch("latent_attention (tensor cores)");
  if (rc || n_splits == 1) return rc;
  const int threads = C >= 128 ? 128 : 64;
  launch_pdl(flint_attn::attention_combine_kernel<__nv_bfloat16>, dim3((unsigned)((long long)T * H)), dim3(threads), 0,
             stream, (const float*)scratch, (__nv_bfloat16*)out, C, n_splits, H, (const int*)nullptr);
  return check_launch("latent_attention (merge)");
}

// out[t, h, :] = W[h] x[t, h, :] for all heads: x [T, H, K] and out [T, H, N] bfloat16 with strides (elements) per
// token and per head, w [H, N, K] bfloat16.  K and the strides of x must be multiples of 8, x and w 16-byte aligned.
extern "C" int flint_head_products(const void* x, long long sx_t, long long sx_h, const void* w, void* out,
                                   long long so_t, long long so_h, int T, int H, int N, int K, cudaStream_t stream) {
  if (T <= 0 || H <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (sx_t & 7) || (sx_h & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return fail("head_products: K=%d and the strides of x must be multiples of 8, x and w 16-byte aligned", K);
  if (H > 65535 || (N + HP_N - 1) / HP_N > 65535) return fail("head_products: too many heads or outputs");
  if (T <= HPS_T && (size_t)T * K * sizeof(float) <= 48 * 1024) {
    launch_pdl(head_products_small_kernel, dim3((N + 7) / 8, H), dim3(256), (size_t)T * K * sizeof(float), stream,
               (const __nv_bfloat16*)x, sx_t, sx_h, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, so_t, so_h, T, N, K);
    return check_launch("head_products (few tokens)");
  }
  dim3 grid((T + HP_M - 1) / HP_M, (N + HP_N - 1) / HP_N, H);
  launch_pdl(head_products_kernel, grid, dim3(128), 0, stream, (const __nv_bfloat16*)x, sx_t, sx_h,
             (const __nv_bfloat16*)w, (__nv_bfloat16*)out, so_t, so_h, T, N, K);
  return check_launch("head_products");
}

extern "C" const char* flint_latent_last_error() { return g_error; }
