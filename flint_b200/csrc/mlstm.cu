// The mLSTM matrix memory as a recurrence over the tokens of a step, in float32.
//
// Per head, with log gates i and f, a running maximum m (from 0), S [D, V] and n [D] (from 0):
//   m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;  n' = e^(f + m - m') n + e^(i - m') k;
//   o  = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)
//
// Three kernels.  flint_mlstm_prepare adds up the partial sums of the input projection [q | k | v | g | z_i | z_f]
// and turns them into what the recurrence reads: q times D^(-1/2), i = cap tanh((z_i + b_i) / cap),
// f = logsigmoid(cap tanh((z_f + b_f) / cap)); it is parallel over tokens.  flint_mlstm_scan walks the tokens of
// every request in order, in two kernels: one block per (request, head), a thread per dim of n, carries m and n and
// leaves every token's decay, intake and denominator; then a warp per CW columns of one head's S (lane l holds rows l, l + 32, ... of
// each) carries those columns, so no warp touches another's part of the state; a block stages the operands of eight
// tokens at a time in shared memory by asynchronous copies, two stages alternating, so the walk does not wait
// for global memory.  The state is read from and written back to the request's row of the state slab
// (per head: S transposed [V, D], then n [D], then m), so a prompt cut anywhere gives the same numbers.
// flint_mlstm_finish divides each head's o by its root mean square and applies the scale and the output gate.
//
// The reference has no mLSTM; its recurrent family keeps state per sequence slot in the same way
// (crates/thuban_architectures/src/qwen35/state.rs:5-55).
#include <math.h>
#include <stdarg.h>
#include "common.cuh"

using namespace flint;

namespace {

constexpr int CW = 2;          // columns of S per warp
constexpr int SCAN_WARPS = 8;  // warps per block of the scan: two to a scheduler hide each other's latencies
constexpr int TCH = 8;         // tokens staged in shared memory at a time (two such stages alternate); at most 32
static_assert(TCH * CW <= 32 && SCAN_WARPS * 32 >= 256, "the gate scan gives a lane a token and a thread a dim (up to 256)");

// Both scans walk a request's tokens one after the other, and what they read of a token does not depend on the
// token before.  A block therefore brings the operands of TCH tokens into shared memory with all its threads
// (q and k of the head, and whatever `more` adds) by asynchronous copies, into one of two stages, while the
// recurrence runs on the other: the walk never waits for global memory at a token.
__device__ __forceinline__ void copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

template <typename More>
__device__ __forceinline__ void stage_tokens(const float* __restrict__ x, int N, int t_first, int n, int oq, int ok, int D,
                                             float* q_s, float* k_s, More more) {
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float* col = x + (size_t)t_first * N + d;
#pragma unroll
    for (int j = 0; j < TCH; ++j)
      if (j < n) {
        copy4(q_s + j * D + d, col + (size_t)j * N + oq);
        copy4(k_s + j * D + d, col + (size_t)j * N + ok);
      }
  }
  more();
  copies_commit();
}

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// x[t, c] = f(sum_z partials[z][t, c]); N = 2 H D + 2 H V + 2 H columns
__global__ void mlstm_prepare_kernel(const float* __restrict__ partials, int S, long long stride,
                                     const float* __restrict__ b_gates, float* __restrict__ x, long long n, int N,
                                     int H, int D, int V, float cap, float q_scale) {
  pdl_launch();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = (int)(i % N);
  float v = 0.f;
  for (int z = 0; z < S; ++z) v += partials[(size_t)z * stride + i];
  const int gates0 = 2 * H * D + 2 * H * V;
  if (c < H * D) {
    v *= q_scale;
  } else if (c >= gates0) {
    const float z = cap * tanhf((v + b_gates[c - gates0]) / cap);
    v = c < gates0 + H ? z : log_sigmoid(z);
  }
  x[i] = v;
}

// The part of the recurrence that all columns of a head share: m, n and the denominator.  One block per (request,
// head), one thread per dim of n (D <= blockDim).  Per staged chunk: every thread walks the short chain of maxima;
// lanes 0 .. TCH - 1 of each warp take a token each and make its decay e^(f + m - m'), intake e^(i - m') and
// e^(-m') (shared by shuffle); every thread carries its dim of n through the chunk; the partial dot products n' . q
// of all tokens are summed side by side over the warp, then over the warps in a fixed order.  The block leaves decay,
// intake and the denominator max(|n' . q|, e^(-m')) + 1e-6 per token in coef [T, H, 4]; it alone touches n and m.
__global__ void __launch_bounds__(SCAN_WARPS * 32)
mlstm_gate_scan_kernel(const float* __restrict__ x, int N, const int* __restrict__ slot, const int* __restrict__ seq_start,
                       int n_seq, float* __restrict__ state, long long state_stride, float* __restrict__ coef, int H,
                       int D, int V) {
  extern __shared__ float sm[];
  const int stage_floats = 2 * TCH * D + 2 * TCH;       // per stage: q [TCH][D], k [TCH][D], log gates [TCH][2]
  __shared__ float part[SCAN_WARPS][TCH];
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, d = threadIdx.x;
  const int h = blockIdx.x % H, e = blockIdx.x / H;
  const int t0 = seq_start ? seq_start[e] : e, t1 = seq_start ? seq_start[e + 1] : e + 1;
  if (t1 <= t0) return;
  float* st = state + (size_t)slot[t0] * state_stride + (size_t)h * ((size_t)D * V + D + 1) + (size_t)D * V;
  float nv = d < D ? st[d] : 0.f;
  float m = st[D];
  const int oq = h * D, ok = H * D + h * D, oi = 2 * H * D + 2 * H * V + h;
  auto stage = [&](int tc, int which) {
    float* q_s = sm + which * stage_floats;
    float* g_s = q_s + 2 * TCH * D;
    const int n = min(TCH, t1 - tc);
    stage_tokens(x, N, tc, n, oq, ok, D, q_s, q_s + TCH * D, [&] {
      for (int j = threadIdx.x; j < 2 * n; j += blockDim.x) copy4(g_s + j, x + (size_t)(tc + (j >> 1)) * N + oi + (j & 1) * H);
    });
  };
  stage(t0, 0);
  int which = 0;
  for (int tc = t0; tc < t1; tc += TCH, which ^= 1) {
    const int n = min(TCH, t1 - tc);
    if (tc + TCH < t1) {
      stage(tc + TCH, which ^ 1);
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncthreads();
    const float* q_s = sm + which * stage_floats;
    const float* k_s = q_s + TCH * D;
    const float* g_s = k_s + TCH * D;
    // the maxima: m before and after the token this lane takes (lanes TCH and up idle along)
    float m_before = m, m_after = m, gi_mine = 0.f, gf_mine = 0.f;
#pragma unroll
    for (int j = 0; j < TCH; ++j)
      if (j < n) {
        const float gi = g_s[2 * j], gf = g_s[2 * j + 1];
        const float m_new = fmaxf(gf + m, gi);
        if (lane == j) { m_before = m; m_after = m_new; gi_mine = gi; gf_mine = gf; }
        m = m_new;
      }
    const float a_mine = expf(gf_mine + m_before - m_after), b_mine = expf(gi_mine - m_after), em_mine = expf(-m_after);
    float pq[TCH];
#pragma unroll
    for (int j = 0; j < TCH; ++j) {
      const float a = __shfl_sync(0xffffffffu, a_mine, j), b = __shfl_sync(0xffffffffu, b_mine, j);
      pq[j] = 0.f;
      if (j < n && d < D) {
        nv = fmaf(a, nv, b * k_s[j * D + d]);
        pq[j] = nv * q_s[j * D + d];
      }
    }
#pragma unroll
    for (int j = 0; j < TCH; ++j) pq[j] = warp_sum(pq[j]);
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < TCH; ++j) part[warp][j] = pq[j];
    }
    __syncthreads();
    if (warp == 0 && lane < n) {
      float nq = 0.f;
#pragma unroll
      for (int w = 0; w < SCAN_WARPS; ++w) nq += part[w][lane];       // fixed order
      float* c = coef + ((size_t)(tc + lane) * H + h) * 4;
      c[0] = a_mine;
      c[1] = b_mine;
      c[2] = fmaxf(fabsf(nq), em_mine) + 1e-6f;
    }
    __syncthreads();          // the stage just read is refilled two chunks on, `part` by the next chunk
  }
  if (d < D) st[d] = nv;
  if (threadIdx.x == 0) st[D] = m;
}

// The matrix memory itself: a block takes SCAN_WARPS * CW columns of one head's S, a warp CW of them (no other warp
// touches them), lane l rows l, l + 32, ...; per token S' = a S + (b k) v^T and o = S'^T q / denominator, with a, b
// and the denominator from coef.
template <int ND>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
mlstm_scan_kernel(const float* __restrict__ x, int N, const int* __restrict__ slot, const int* __restrict__ seq_start,
                  int n_seq, float* __restrict__ state, long long state_stride, const float* __restrict__ coef,
                  float* __restrict__ out, int H, int D, int V, int col_blocks) {
  constexpr int BC = SCAN_WARPS * CW;    // columns per block
  extern __shared__ float sm[];
  const int stage_floats = 2 * TCH * D + TCH * BC + 4 * TCH;   // per stage: q, k [TCH][D], v [TCH][BC], coef [TCH][4]
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cb = blockIdx.x % col_blocks, h = (blockIdx.x / col_blocks) % H, e = blockIdx.x / (col_blocks * H);
  const int t0 = seq_start ? seq_start[e] : e, t1 = seq_start ? seq_start[e + 1] : e + 1;
  if (t1 <= t0) return;
  float* st = state + (size_t)slot[t0] * state_stride + (size_t)h * ((size_t)D * V + D + 1);
  const int c0 = cb * BC + warp * CW;
  float Sm[CW][ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
#pragma unroll
    for (int c = 0; c < CW; ++c) Sm[c][i] = (d < D && c0 + c < V) ? st[(size_t)(c0 + c) * D + d] : 0.f;
  }
  const int oq = h * D, ok = H * D + h * D, ov = 2 * H * D + h * V + cb * BC;
  // columns beyond the head's last have the value 0 in both stages, once and for all
  for (int j = threadIdx.x; j < 2 * TCH * BC; j += blockDim.x)
    if (cb * BC + j % BC >= V) sm[(j / (TCH * BC)) * stage_floats + 2 * TCH * D + j % (TCH * BC)] = 0.f;
  auto stage = [&](int tc, int which) {
    float* q_s = sm + which * stage_floats;
    float* v_s = q_s + 2 * TCH * D;
    float* c_s = v_s + TCH * BC;
    const int n = min(TCH, t1 - tc);
    stage_tokens(x, N, tc, n, oq, ok, D, q_s, q_s + TCH * D, [&] {
      for (int j = threadIdx.x; j < n * BC; j += blockDim.x)
        if (cb * BC + j % BC < V) copy4(v_s + j, x + (size_t)(tc + j / BC) * N + ov + j % BC);
      for (int j = threadIdx.x; j < n * 4; j += blockDim.x) copy4(c_s + j, coef + ((size_t)(tc + (j >> 2)) * H + h) * 4 + (j & 3));
    });
  };
  stage(t0, 0);
  int which = 0;
  for (int tc = t0; tc < t1; tc += TCH, which ^= 1) {
    const int n = min(TCH, t1 - tc);
    if (tc + TCH < t1) {
      stage(tc + TCH, which ^ 1);
      copies_wait<1>();
    } else {
      copies_wait<0>();
    }
    __syncthreads();
    const float* q_s = sm + which * stage_floats;
    const float* k_s = q_s + TCH * D;
    const float* v_s = k_s + TCH * D;
    const float* c_s = v_s + TCH * BC;
    if (c0 < V) {
      // the chunk's tokens one after the other through S (a chain of one multiply-add a token and element); the
      // sums over the warp of all tokens and columns then run side by side, and lane j CW + c writes token j's column c
      float acc[TCH][CW];
#pragma unroll
      for (int j = 0; j < TCH; ++j) {
#pragma unroll
        for (int c = 0; c < CW; ++c) acc[j][c] = 0.f;
        if (j < n) {
          const float a = c_s[4 * j], b = c_s[4 * j + 1];
          float v[CW];
#pragma unroll
          for (int c = 0; c < CW; ++c) v[c] = v_s[j * BC + warp * CW + c];
#pragma unroll
          for (int i = 0; i < ND; ++i) {
            const int d = lane + 32 * i;
            const float kd = d < D ? k_s[j * D + d] : 0.f, qd = d < D ? q_s[j * D + d] : 0.f;
            const float bk = b * kd;
#pragma unroll
            for (int c = 0; c < CW; ++c) {
              Sm[c][i] = fmaf(a, Sm[c][i], bk * v[c]);
              acc[j][c] = fmaf(Sm[c][i], qd, acc[j][c]);
            }
          }
        }
      }
      float mine = 0.f;
#pragma unroll
      for (int j = 0; j < TCH; ++j)
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          const float t = warp_sum(acc[j][c]);
          mine = lane == j * CW + c ? t : mine;
        }
      const int j = lane / CW, c = lane % CW;
      if (j < n && c0 + c < V) out[((size_t)(tc + j) * H + h) * V + c0 + c] = mine / c_s[4 * j + 2];
    }
    __syncthreads();          // the stage just read is refilled two chunks on
  }
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < D) {
#pragma unroll
      for (int c = 0; c < CW; ++c)
        if (c0 + c < V) st[(size_t)(c0 + c) * D + d] = Sm[c][i];
    }
  }
}

// out[t, h, c] = o[t, h, c] / sqrt(mean_c o[t, h, :]^2 + eps) * w[h V + c] * sigmoid(gate[t, h V + c]); a warp per (t, h)
template <typename TO>
__global__ void mlstm_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long gate_stride,
                                    const float* __restrict__ w, float eps, TO* __restrict__ out, long long n_items,
                                    int H, int V) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const long long t = item / H;
  const int h = (int)(item % H);
  const float* row = o + ((size_t)t * H + h) * V;
  float ss = 0.f;
  for (int c = lane; c < V; c += 32) ss = fmaf(row[c], row[c], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)V + eps);
  for (int c = lane; c < V; c += 32) {
    const float g = gate[(size_t)t * gate_stride + (size_t)h * V + c];
    out[((size_t)t * H + h) * V + c] = from_f32<TO>(row[c] * inv * w[(size_t)h * V + c] * (1.0f / (1.0f + expf(-g))));
  }
}

}  // namespace

// partials [S, T, N] float32 -> x [T, N] float32 (see the top of the file); N = 2 H D + 2 H V + 2 H.
extern "C" int flint_mlstm_prepare(const float* partials, int S, long long stride, const float* b_gates, float* x,
                                   int T, int H, int D, int V, float cap, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (S < 1) return fail("mlstm_prepare: needs at least one partial");
  if (H < 1 || D < 1 || V < 1 || !(cap > 0.f)) return fail("mlstm_prepare: bad sizes (%d heads, %d, %d) or gate cap", H, D, V);
  const int N = 2 * H * D + 2 * H * V + 2 * H;
  const long long n = (long long)T * N;
  launch_pdl(mlstm_prepare_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, partials, S, stride, b_gates,
             x, n, N, H, D, V, cap, 1.0f / sqrtf((float)D));
  return check_launch("mlstm_prepare");
}

// x [T, N] as flint_mlstm_prepare leaves it; the rows of request e are seq_start[e] .. seq_start[e + 1] - 1 (NULL:
// row e alone); state [slots, state_stride] float32; coef [T, H, 4] float32 scratch; out [T, H V] float32.
extern "C" int flint_mlstm_scan(const float* x, const int* slot, const int* seq_start, int n_seq, float* state,
                                long long state_stride, float* coef, float* out, int T, int H, int D, int V,
                                cudaStream_t stream) {
  if (T <= 0 || n_seq <= 0) return 0;
  if (H < 1 || D < 1 || V < 1 || D > 256) return fail("mlstm_scan: %d heads of %d x %d are not supported (dims up to 256)", H, D, V);
  if (state_stride < (long long)H * ((long long)D * V + D + 1)) return fail("mlstm_scan: the state rows are too short");
  if (!seq_start && n_seq != T) return fail("mlstm_scan: without a list of starts every request brings one row");
  const int N = 2 * H * D + 2 * H * V + 2 * H;
  const int col_blocks = (V + SCAN_WARPS * CW - 1) / (SCAN_WARPS * CW);
  const long long gate_blocks = (long long)n_seq * H, blocks = gate_blocks * col_blocks;
  if (blocks > 0x7fffffffLL) return fail("mlstm_scan: too many work items");
  const dim3 gate_grid((unsigned)gate_blocks), grid((unsigned)blocks), block(SCAN_WARPS * 32);
  const size_t gate_smem = (size_t)2 * (2 * TCH * D + 2 * TCH) * sizeof(float);                      // two stages each
  const size_t smem = (size_t)2 * (2 * TCH * D + TCH * SCAN_WARPS * CW + 4 * TCH) * sizeof(float);
#define SCAN(ND)                                                                                                     \
  do {                                                                                                               \
    launch_pdl(mlstm_gate_scan_kernel, gate_grid, block, gate_smem, stream, x, N, slot, seq_start, n_seq, state,     \
               state_stride, coef, H, D, V);                                                                         \
    launch_pdl(mlstm_scan_kernel<ND>, grid, block, smem, stream, x, N, slot, seq_start, n_seq, state, state_stride,  \
               (const float*)coef, out, H, D, V, col_blocks);                                                        \
  } while (0)
  if (D <= 32) SCAN(1);
  else if (D <= 64) SCAN(2);
  else if (D <= 128) SCAN(4);
  else SCAN(8);
#undef SCAN
  return check_launch("mlstm_scan");
}

extern "C" int flint_mlstm_finish(const float* o, const float* gate, long long gate_stride, const float* w, float eps,
                                  void* out, int out_dtype, int T, int H, int V, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long items = (long long)T * H;
  FLINT_DISPATCH_DTYPE(out_dtype, TO,
      launch_pdl(mlstm_finish_kernel<TO>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, o, gate, gate_stride, w,
                 eps, (TO*)out, items, H, V));
  return check_launch("mlstm_finish");
}

extern "C" const char* flint_mlstm_last_error() { return g_error; }
