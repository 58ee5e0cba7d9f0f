// A feed-forward of routed experts: every token goes through `top` of E small gated feed-forwards.
//
//   1. sb_moe_route: from float router logits [T, E], the `top` largest scores of every token (sigmoid or softmax
//      scores; lowest index on ties) and their weights, as float.
//   2. sb_moe_sort: the (token, choice) pairs grouped by expert: offsets[E + 1] and the pairs in that order, plus
//      the list of row tiles (expert, first row) the products run over. Which place a pair gets inside its
//      expert's group depends on timing, but nothing computed from it does: a pair's result is a function of its
//      own row alone.
//   3. sb_moe_gate_up: act[row] = f( w * (x W_gate^T), w * (x W_up^T) ) for the rows of every tile, x the pair's
//      token. The weight multiplies the expert's input; a product is linear, so it is applied to the float sums.
//   4. sb_moe_down: out[pair] = act[row] W_down^T, written at the pair's own place; with top == 1 that is the result,
//      otherwise sb_moe_combine adds a token's `top` rows in order.
// Products accumulate in float over k in ascending order, whatever else is in the step.
#include "common.cuh"

using namespace sb;

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

constexpr int ROUTE_MAX_TOP = 16;

// One thread per token: E is small, and the scores are read once.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int E, int top, int score_kind, int renorm,
                                                        int n_tokens, int* __restrict__ idx, float* __restrict__ wts) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * E;
  int best[ROUTE_MAX_TOP];
  float val[ROUTE_MAX_TOP];
  float zmax = -INFINITY, denom = 1.f;
  if (score_kind == 1) {                        // softmax over all experts
    for (int e = 0; e < E; ++e) zmax = fmaxf(zmax, z[e]);
    denom = 0.f;
    for (int e = 0; e < E; ++e) denom += expf(z[e] - zmax);
  }
  for (int s = 0; s < top; ++s) {
    int arg = -1;
    float m = -INFINITY;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int u = 0; u < s; ++u) taken |= best[u] == e;
      if (!taken && (arg < 0 || z[e] > m)) { m = z[e]; arg = e; }      // the scores are monotone in the logits
    }
    best[s] = arg;
    val[s] = score_kind == 1 ? expf(m - zmax) / denom : sigmoid_f(m);
  }
  float total = 0.f;
  for (int s = 0; s < top; ++s) total += val[s];
  for (int s = 0; s < top; ++s) {
    idx[(size_t)t * top + s] = best[s];
    wts[(size_t)t * top + s] = renorm ? val[s] / total : val[s];
  }
}

constexpr int TM = 32;            // rows of a tile

// One block. order[offsets[e] .. offsets[e+1]) = the pairs of expert e; tiles: (expert, first row) for every TM rows
// of an expert's group, n_tiles[0] of them.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int E, int* __restrict__ offsets,
                                                        int* __restrict__ order, int* __restrict__ tiles, int* __restrict__ n_tiles) {
  extern __shared__ int sh[];
  int* count = sh;            // [E]
  int* start = sh + E;        // [E + 1]
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      offsets[e] = at;
      for (int r0 = 0; r0 < count[e]; r0 += TM) {
        tiles[2 * nt] = e;
        tiles[2 * nt + 1] = at + r0;
        ++nt;
      }
      at += count[e];
    }
    start[E] = at;
    offsets[E] = at;
    n_tiles[0] = nt;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < E) order[start[e] + atomicAdd(&count[e], 1)] = p;
  }
}

constexpr int TK = 32;
constexpr int GU_COLS = 32;       // gate columns of a tile (and as many up columns)
constexpr int DN_COLS = 64;
constexpr int MOE_THREADS = 256;

// grid (column tiles of ff, row tiles). x [T, K] with row stride; w_gu [E, 2 ff, K] (gate rows, then up rows).
// act kinds: 0 = silu(g) * u; 1 = the clamped form: g <- min(g, limit), u <- clamp(u, -limit, limit), g * sigmoid(alpha g) * (u + 1).
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS) moe_gate_up_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ w_gu,
                                                                  const int* __restrict__ order, const int* __restrict__ offsets,
                                                                  const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                                  const float* __restrict__ wts, int top, int K, int ff, int scale_input,
                                                                  int act_kind, float limit, float alpha, T* __restrict__ act) {
  if ((int)blockIdx.y >= n_tiles[0]) return;
  __shared__ float As[TK][TM + 1];
  __shared__ float Bg[TK][GU_COLS + 1];
  __shared__ float Bu[TK][GU_COLS + 1];
  __shared__ int tok[TM];
  __shared__ float rw[TM];
  const int e = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
  const int rows = min(TM, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * GU_COLS;
  const int tid = threadIdx.x;
  if (tid < TM) {
    const int pair = tid < rows ? order[row0 + tid] : -1;
    tok[tid] = pair >= 0 ? pair / top : -1;
    rw[tid] = pair >= 0 ? wts[pair] : 0.f;
  }
  __syncthreads();
  const T* wg = w_gu + (size_t)e * 2 * ff * K;
  const T* wu = wg + (size_t)ff * K;
  const int ty = tid >> 4, tx = tid & 15;               // rows 2 ty, 2 ty + 1; columns 2 tx, 2 tx + 1
  float ag[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, au[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int w = tid; w < TM * TK; w += MOE_THREADS) {
      const int m = w / TK, kk = w - m * TK;
      const int tk = tok[m];
      As[kk][m] = (tk >= 0 && k0 + kk < K) ? to_float(x[(size_t)tk * x_stride + k0 + kk]) : 0.f;
    }
    for (int w = tid; w < GU_COLS * TK; w += MOE_THREADS) {
      const int nn = w / TK, kk = w - nn * TK;
      const bool ok = n0 + nn < ff && k0 + kk < K;
      Bg[kk][nn] = ok ? to_float(wg[(size_t)(n0 + nn) * K + k0 + kk]) : 0.f;
      Bu[kk][nn] = ok ? to_float(wu[(size_t)(n0 + nn) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = As[kk][2 * ty], a1 = As[kk][2 * ty + 1];
      const float g0 = Bg[kk][2 * tx], g1 = Bg[kk][2 * tx + 1], u0 = Bu[kk][2 * tx], u1 = Bu[kk][2 * tx + 1];
      ag[0][0] += a0 * g0; ag[0][1] += a0 * g1; ag[1][0] += a1 * g0; ag[1][1] += a1 * g1;
      au[0][0] += a0 * u0; au[0][1] += a0 * u1; au[1][0] += a1 * u0; au[1][1] += a1 * u1;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = 2 * ty + i;
    if (m >= rows) continue;
    const float sc = scale_input ? rw[m] : 1.f;
#pragma unroll
    for (int jx = 0; jx < 2; ++jx) {
      const int nn = n0 + 2 * tx + jx;
      if (nn >= ff) continue;
      float g = ag[i][jx] * sc, u = au[i][jx] * sc, yv;
      if (act_kind == 1) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        yv = g * sigmoid_f(alpha * g) * (u + 1.f);
      } else {
        yv = g * sigmoid_f(g) * u;
      }
      act[(size_t)(row0 + m) * ff + nn] = from_float<T>(yv);
    }
  }
}

// grid (column tiles of N, row tiles). act [rows, ff]; w_down [E, N, ff]; out [pairs, N] at the pair's own place, each
// row times its weight unless the weight already went into the input.
template <typename T, typename O>
__global__ void __launch_bounds__(MOE_THREADS) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down,
                                                               const int* __restrict__ order, const int* __restrict__ offsets,
                                                               const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                               const float* __restrict__ wts, int ff, int N, int scale_output,
                                                               O* __restrict__ out) {
  if ((int)blockIdx.y >= n_tiles[0]) return;
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][DN_COLS + 1];
  __shared__ int pair_of[TM];
  const int e = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
  const int rows = min(TM, offsets[e + 1] - row0);
  const int n0 = blockIdx.x * DN_COLS;
  const int tid = threadIdx.x;
  if (tid < TM) pair_of[tid] = tid < rows ? order[row0 + tid] : -1;
  __syncthreads();
  const T* w = w_down + (size_t)e * N * ff;
  const int ty = tid >> 4, tx = tid & 15;               // rows 2 ty, 2 ty + 1; columns tx, tx + 16, tx + 32, tx + 48
  float acc[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int jx = 0; jx < 4; ++jx) acc[i][jx] = 0.f;
  for (int k0 = 0; k0 < ff; k0 += TK) {
    for (int v = tid; v < TM * TK; v += MOE_THREADS) {
      const int m = v / TK, kk = v - m * TK;
      As[kk][m] = (m < rows && k0 + kk < ff) ? to_float(act[(size_t)(row0 + m) * ff + k0 + kk]) : 0.f;
    }
    for (int v = tid; v < DN_COLS * TK; v += MOE_THREADS) {
      const int nn = v / TK, kk = v - nn * TK;
      Bs[kk][nn] = (n0 + nn < N && k0 + kk < ff) ? to_float(w[(size_t)(n0 + nn) * ff + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = As[kk][2 * ty], a1 = As[kk][2 * ty + 1];
#pragma unroll
      for (int jx = 0; jx < 4; ++jx) {
        const float b = Bs[kk][tx + 16 * jx];
        acc[0][jx] += a0 * b;
        acc[1][jx] += a1 * b;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = 2 * ty + i;
    if (m >= rows) continue;
    const int pair = pair_of[m];
    const float sc = scale_output ? wts[pair] : 1.f;
#pragma unroll
    for (int jx = 0; jx < 4; ++jx) {
      const int nn = n0 + tx + 16 * jx;
      if (nn < N) out[(size_t)pair * N + nn] = from_float<O>(acc[i][jx] * sc);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ parts, int top, int N, long long total,
                                                          T* __restrict__ out) {
  for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
    const long long t = w / N;
    const int c = (int)(w - t * N);
    float s = 0.f;
    for (int k = 0; k < top; ++k) s += parts[((size_t)t * top + k) * N + c];
    out[w] = from_float<T>(s);
  }
}

}  // namespace

SB_EXPORT int sb_moe_tile_rows() { return TM; }

// logits float [T, E] -> idx int32 [T, top], wts float [T, top]. score_kind 0: sigmoid of the logit, 1: softmax over the
// experts; renorm: the chosen weights divided by their sum.
SB_EXPORT int sb_moe_route(const float* logits, int E, int top, int score_kind, int renorm, int n_tokens, int* idx, float* wts,
                           cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || top > ROUTE_MAX_TOP) return SB_ERR_LIMIT;
  moe_route_kernel<<<(n_tokens + 127) / 128, 128, 0, stream>>>(logits, E, top, score_kind, renorm, n_tokens, idx, wts);
  SB_LAUNCH_CHECK();
  return 0;
}

// idx int32 [n_pairs] -> offsets [E + 1], order [n_pairs], tiles [2 * (n_pairs / TM + E)], n_tiles [1].
SB_EXPORT int sb_moe_sort(const int* idx, int n_pairs, int E, int* offsets, int* order, int* tiles, int* n_tiles, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (E <= 0 || E > 4096) return SB_ERR_LIMIT;
  moe_sort_kernel<<<1, 1024, (size_t)(2 * E + 1) * sizeof(int), stream>>>(idx, n_pairs, E, offsets, order, tiles, n_tiles);
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_moe_gate_up(const void* x, int x_stride, const void* w_gu, const int* order, const int* offsets, const int* tiles,
                             const int* n_tiles, const float* wts, int top, int n_pairs, int E, int K, int ff, int scale_input,
                             int act_kind, float limit, float alpha, void* act, int dtype, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  const int max_tiles = n_pairs / TM + (E < n_pairs ? E : n_pairs);
  if (max_tiles > 65535) return SB_ERR_LIMIT;
  dim3 grid((ff + GU_COLS - 1) / GU_COLS, max_tiles);
  if (dtype == SB_DTYPE_F32)
    moe_gate_up_kernel<float><<<grid, MOE_THREADS, 0, stream>>>((const float*)x, x_stride, (const float*)w_gu, order, offsets, tiles,
                                                                 n_tiles, wts, top, K, ff, scale_input, act_kind, limit, alpha, (float*)act);
  else if (dtype == SB_DTYPE_BF16)
    moe_gate_up_kernel<__nv_bfloat16><<<grid, MOE_THREADS, 0, stream>>>((const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)w_gu,
                                                                         order, offsets, tiles, n_tiles, wts, top, K, ff, scale_input,
                                                                         act_kind, limit, alpha, (__nv_bfloat16*)act);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// out: [n_pairs, N] of dtype out_dtype (float for rows that are still to be added up).
SB_EXPORT int sb_moe_down(const void* act, const void* w_down, const int* order, const int* offsets, const int* tiles, const int* n_tiles,
                          const float* wts, int n_pairs, int E, int ff, int N, int scale_output, void* out, int dtype, int out_dtype,
                          cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  const int max_tiles = n_pairs / TM + (E < n_pairs ? E : n_pairs);
  if (max_tiles > 65535) return SB_ERR_LIMIT;
  dim3 grid((N + DN_COLS - 1) / DN_COLS, max_tiles);
  if (dtype == SB_DTYPE_F32 && out_dtype == SB_DTYPE_F32)
    moe_down_kernel<float, float><<<grid, MOE_THREADS, 0, stream>>>((const float*)act, (const float*)w_down, order, offsets, tiles, n_tiles,
                                                                     wts, ff, N, scale_output, (float*)out);
  else if (dtype == SB_DTYPE_BF16 && out_dtype == SB_DTYPE_BF16)
    moe_down_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, MOE_THREADS, 0, stream>>>(
        (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, order, offsets, tiles, n_tiles, wts, ff, N, scale_output,
        (__nv_bfloat16*)out);
  else if (dtype == SB_DTYPE_BF16 && out_dtype == SB_DTYPE_F32)
    moe_down_kernel<__nv_bfloat16, float><<<grid, MOE_THREADS, 0, stream>>>((const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, order,
                                                                             offsets, tiles, n_tiles, wts, ff, N, scale_output, (float*)out);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

// parts float [T * top, N] -> out [T, N]: a token's rows added in the order of its choices.
SB_EXPORT int sb_moe_combine(const float* parts, int top, int n_tokens, int N, void* out, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const long long total = (long long)n_tokens * N;
  const long long want = (total + 255) / 256;
  const int blocks = (int)(want < sm_count() * 8 ? want : sm_count() * 8);
  if (dtype == SB_DTYPE_F32) moe_combine_kernel<float><<<blocks, 256, 0, stream>>>(parts, top, N, total, (float*)out);
  else if (dtype == SB_DTYPE_BF16) moe_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(parts, top, N, total, (__nv_bfloat16*)out);
  else return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}
