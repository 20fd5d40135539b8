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

extern "C" const char* flint_latent_last_error() { return g_error; }
