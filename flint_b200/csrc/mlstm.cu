// The mLSTM matrix memory as a recurrence over the tokens of a step, in float32.
//
// Per head, with log gates i and f, a running maximum m (from 0), S [D, V] and n [D] (from 0):
//   m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;  n' = e^(f + m - m') n + e^(i - m') k;
//   o  = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)
//
// Three kernels.  flint_mlstm_prepare adds up the partial sums of the input projection [q | k | v | g | z_i | z_f]
// and turns them into what the recurrence reads: q times D^(-1/2), i = cap tanh((z_i + b_i) / cap),
// f = logsigmoid(cap tanh((z_f + b_f) / cap)); it is parallel over tokens.  flint_mlstm_scan walks the tokens of
// every request in order, in two kernels: one warp per (request, head) carries m and n and leaves every token's
// decay, intake and denominator; then a warp per CW columns of one head's S (lane l holds rows l, l + 32, ... of
// each) carries those columns, so no warp touches another's part of the state; a block stages the operands of 16
// tokens at a time in shared memory, so the walk does not wait for global memory at every token.  The state is read from and written back to the request's row of the state slab
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

constexpr int CW = 4;          // columns of S per warp
constexpr int SCAN_WARPS = 4;  // warps per block of the scan
constexpr int TCH = 16;        // tokens staged in shared memory at a time

// Both scans walk a request's tokens one after the other, and what they read of a token does not depend on the
// token before.  A block therefore brings the operands of TCH tokens into shared memory with all its threads
// (q and k of the head, and whatever `more` adds), and the recurrence then runs on those without waiting for
// global memory at every token.
template <typename More>
__device__ __forceinline__ void stage_tokens(const float* __restrict__ x, int N, int t_first, int n, int oq, int ok, int D,
                                             float* q_s, float* k_s, More more) {
  // a thread takes dims d, d + blockDim.x, ... of every staged token; the loads of all TCH tokens are in flight
  // together (one after the other they would each cost a trip to L2)
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float tq[TCH], tk[TCH];
    const float* col = x + (size_t)t_first * N + d;
#pragma unroll
    for (int j = 0; j < TCH; ++j) {
      tq[j] = j < n ? col[(size_t)j * N + oq] : 0.f;
      tk[j] = j < n ? col[(size_t)j * N + ok] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < TCH; ++j) {
      q_s[j * D + d] = tq[j];
      k_s[j * D + d] = tk[j];
    }
  }
  more();
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
// head); its first warp walks the request's tokens and leaves, per token, the decay e^(f + m - m'), the intake
// e^(i - m') and the denominator max(|n' . q|, e^(-m')) + 1e-6 in coef [T, H, 4]; it alone reads and writes n and
// m of the state.
template <int ND>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
mlstm_gate_scan_kernel(const float* __restrict__ x, int N, const int* __restrict__ slot, const int* __restrict__ seq_start,
                       int n_seq, float* __restrict__ state, long long state_stride, float* __restrict__ coef, int H,
                       int D, int V) {
  extern __shared__ float sm[];
  float* q_s = sm;                       // [TCH][D]
  float* k_s = q_s + TCH * D;            // [TCH][D]
  float* g_s = k_s + TCH * D;            // [TCH][2]: log input gate, log forget gate
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.x % H, e = blockIdx.x / H;
  const int t0 = seq_start ? seq_start[e] : e, t1 = seq_start ? seq_start[e + 1] : e + 1;
  if (t1 <= t0) return;
  float* st = state + (size_t)slot[t0] * state_stride + (size_t)h * ((size_t)D * V + D + 1) + (size_t)D * V;
  float nv[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) nv[i] = (warp == 0 && lane + 32 * i < D) ? st[lane + 32 * i] : 0.f;
  float m = st[D];
  const int oq = h * D, ok = H * D + h * D, oi = 2 * H * D + 2 * H * V + h;
  for (int tc = t0; tc < t1; tc += TCH) {
    const int n = min(TCH, t1 - tc);
    stage_tokens(x, N, tc, n, oq, ok, D, q_s, k_s, [&] {
      for (int j = threadIdx.x; j < 2 * n; j += blockDim.x) g_s[j] = x[(size_t)(tc + (j >> 1)) * N + oi + (j & 1) * H];
    });
    __syncthreads();
    if (warp == 0) {
      for (int j = 0; j < n; ++j) {
        const float gi = g_s[2 * j], gf = g_s[2 * j + 1];
        const float m_new = fmaxf(gf + m, gi);
        const float a = expf(gf + m - m_new), b = expf(gi - m_new);
        float nq = 0.f;
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          const int d = lane + 32 * i;
          if (d < D) {
            nv[i] = fmaf(a, nv[i], b * k_s[j * D + d]);
            nq = fmaf(nv[i], q_s[j * D + d], nq);
          }
        }
        nq = warp_sum(nq);
        if (lane == 0) {
          float* c = coef + ((size_t)(tc + j) * H + h) * 4;
          c[0] = a;
          c[1] = b;
          c[2] = fmaxf(fabsf(nq), expf(-m_new)) + 1e-6f;
        }
        m = m_new;
      }
    }
    __syncthreads();
  }
  if (warp != 0) return;
#pragma unroll
  for (int i = 0; i < ND; ++i)
    if (lane + 32 * i < D) st[lane + 32 * i] = nv[i];
  if (lane == 0) st[D] = m;
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
  float* q_s = sm;                       // [TCH][D]
  float* k_s = q_s + TCH * D;            // [TCH][D]
  float* v_s = k_s + TCH * D;            // [TCH][BC]
  float* c_s = v_s + TCH * BC;           // [TCH][4]: decay, intake, denominator
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
  for (int tc = t0; tc < t1; tc += TCH) {
    const int n = min(TCH, t1 - tc);
    stage_tokens(x, N, tc, n, oq, ok, D, q_s, k_s, [&] {
      for (int j = threadIdx.x; j < n * BC; j += blockDim.x)
        v_s[j] = cb * BC + j % BC < V ? x[(size_t)(tc + j / BC) * N + ov + j % BC] : 0.f;
      for (int j = threadIdx.x; j < n * 4; j += blockDim.x) c_s[j] = coef[((size_t)(tc + (j >> 2)) * H + h) * 4 + (j & 3)];
    });
    __syncthreads();
    if (c0 < V) {
#pragma unroll 2
      for (int j = 0; j < n; ++j) {
        const float a = c_s[4 * j], b = c_s[4 * j + 1], den = c_s[4 * j + 2];
        float v[CW], acc[CW];
#pragma unroll
        for (int c = 0; c < CW; ++c) {
          v[c] = v_s[j * BC + warp * CW + c];
          acc[c] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          const int d = lane + 32 * i;
          const float kd = d < D ? k_s[j * D + d] : 0.f, qd = d < D ? q_s[j * D + d] : 0.f;
          const float bk = b * kd;
#pragma unroll
          for (int c = 0; c < CW; ++c) {
            Sm[c][i] = fmaf(a, Sm[c][i], bk * v[c]);
            acc[c] = fmaf(Sm[c][i], qd, acc[c]);
          }
        }
#pragma unroll
        for (int c = 0; c < CW; ++c) acc[c] = warp_sum(acc[c]);
        float mine = acc[0];
#pragma unroll
        for (int c = 1; c < CW; ++c) mine = lane == c ? acc[c] : mine;
        if (lane < CW && c0 + lane < V) out[((size_t)(tc + j) * H + h) * V + c0 + lane] = mine / den;
      }
    }
    __syncthreads();
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
  const size_t gate_smem = (size_t)(2 * TCH * D + 2 * TCH) * sizeof(float);
  const size_t smem = (size_t)(2 * TCH * D + TCH * SCAN_WARPS * CW + 4 * TCH) * sizeof(float);
#define SCAN(ND)                                                                                                     \
  do {                                                                                                               \
    launch_pdl(mlstm_gate_scan_kernel<ND>, gate_grid, block, gate_smem, stream, x, N, slot, seq_start, n_seq, state, \
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
