// Kernels of mixers that carry a state of fixed size from token to token instead of (or beside) cached keys:
// short causal convolutions over time, linear recurrences over a matrix state per head (fixed decay, selective
// state space, gated delta rule), the normalisation-and-gate that follows them, and the cache write of an
// attention whose values are normalised and whose queries and keys are not rotated.
//
// A step is ragged: row r brings the tokens cu_q[r] .. cu_q[r+1]-1 and owns state slot slots[r]. State tensors
// are float [max_slots, ...] and are zero when a slot is handed out, so "zeros before the start" needs no
// special case: a request's first portion reads the zeros, every later portion what the one before left.
// Everything that enters a recurrence is float, in both dtypes; activations read and written are T.
#include "common.cuh"

using namespace sb;

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float load_w(const void* p, int dtype, size_t i) {
  return dtype == SB_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// ------------------------------------------------------------------------------------------ short convolution
// out[t, c] = act( bias[c] + sum_j w[c, j] * in[t - taps + 1 + j, c]  (+ in[t, c] if residual) ), in[-1], in[-2], ...
// of a row's first token being the inputs the state holds: state[slot, m, c] is the input taps - 1 - m tokens
// before the portion's start. With inline_state (every row brings one token) the thread also shifts the state.
constexpr int CONV_THREADS = 128;
constexpr int CONV_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS) causal_conv_kernel(
    const T* __restrict__ x, int x_stride, const T* __restrict__ w, const T* __restrict__ bias, float* __restrict__ state,
    const int* __restrict__ slots, const int* __restrict__ cu_q, const int* __restrict__ token_row, T* __restrict__ out,
    int out_stride, int C, int taps, int act, int residual, int inline_state) {
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  const int t = blockIdx.y;
  if (c >= C) return;
  const int r = token_row[t];
  const int i = t - cu_q[r];
  const int K = taps - 1;
  float* st = state + (size_t)slots[r] * K * C + c;
  float acc = bias ? to_float(bias[c]) : 0.f;
  float cur = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = i - K + j;
    const float v = src >= 0 ? to_float(x[(size_t)(t - K + j) * x_stride + c]) : st[(size_t)(K + src) * C];
    acc += to_float(w[(size_t)c * taps + j]) * v;
    cur = v;
  }
  if (residual) acc += cur;
  if (act == 1) acc = silu_f(acc);
  out[(size_t)t * out_stride + c] = from_float<T>(acc);
  if (inline_state) {
    for (int m = 0; m + 1 < K; ++m) st[(size_t)m * C] = st[(size_t)(m + 1) * C];
    if (K > 0) st[(size_t)(K - 1) * C] = cur;
  }
}

// After a step: the state of row r becomes its last taps - 1 inputs (older ones come from the old state when the
// portion is shorter than that). One thread per (row, channel) reads all it needs before it writes.
template <typename T>
__global__ void __launch_bounds__(CONV_THREADS) conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state,
                                                                   const int* __restrict__ slots, const int* __restrict__ cu_q, int C,
                                                                   int taps) {
  const int c = blockIdx.x * CONV_THREADS + threadIdx.x;
  const int r = blockIdx.y;
  if (c >= C) return;
  const int q0 = cu_q[r], n = cu_q[r + 1] - q0;
  const int K = taps - 1;
  float* st = state + (size_t)slots[r] * K * C + c;
  float keep[CONV_MAX_TAPS];
#pragma unroll
  for (int m = 0; m < CONV_MAX_TAPS; ++m) {
    if (m < K) {
      const int src = n - K + m;                        // index among the portion's tokens
      keep[m] = src >= 0 ? to_float(x[(size_t)(q0 + src) * x_stride + c]) : st[(size_t)(m + n) * C];
    }
  }
#pragma unroll
  for (int m = 0; m < CONV_MAX_TAPS; ++m)
    if (m < K) st[(size_t)m * C] = keep[m];
}

// ------------------------------------------------------------------------------------------ linear recurrences
// One state matrix S [dk, dv] per (request, head); per token, with a decay a (a number, or one per row of S):
//   S <- a * S;   u = v                      (MODE_DECAY, MODE_SSM: u = dt * x)
//                 u = beta * (v - S^T k)     (MODE_DELTA)
//   S <- S + k u^T;   o = S^T q  (+ D * x for MODE_SSM)
// The columns of S never meet, so a block takes (request, head, a slice of columns) and walks the row's tokens in
// order. A thread keeps REC_RPT rows of one column in registers (rows part, part + P, ...; P lanes share a column
// and add their parts by shuffles), so dk <= 32 * REC_RPT. Tokens are staged through shared memory REC_TS at a
// time; what each mode does to its inputs on the way (silu; softplus and exponentials; unit vectors) happens
// there, in float.
constexpr int MODE_DECAY = 0, MODE_SSM = 1, MODE_DELTA = 2;
constexpr int REC_RPT = 16;
constexpr int REC_WARPS = 4;
constexpr int REC_THREADS = REC_WARPS * 32;

struct RecArgs {
  const void* q; const void* k; const void* v;      // [T, *] activations: row strides below, head h at h * dk (dv)
  int q_stride, k_stride, v_stride;
  const void* aux;  int aux_stride;                  // SSM: dt before softplus [T, H]; DELTA: beta before the sigmoid [T, H]
  const void* rate; int rate_stride;                 // DELTA: decay rate before softplus [T, H * dk]
  const void* decay;                                 // DECAY: [H] float decays
  const void* a_log; const void* dt_bias; const void* d_skip;   // parameters (dtype par_dtype)
  int par_dtype;
  float* state;                                      // [slots, H, dk, dv]
  const int* slots; const int* cu_q;
  float* out; int out_stride;                        // [T, H * dv] float
  int H, Hqk, dk, dv, P, ts;
  float q_scale;
};

template <typename T, int MODE>
__global__ void __launch_bounds__(REC_THREADS) recurrence_kernel(RecArgs a) {
  extern __shared__ float smem[];
  const int dk = a.dk, dv = a.dv, P = a.P, TS = a.ts;
  const int VC = REC_THREADS / P;                       // columns of this block
  float* qs = smem;                                     // [TS][dk]
  float* ks = qs + TS * dk;                             // [TS][dk]
  float* vs = ks + TS * dk;                             // [TS][VC]
  float* as = vs + TS * VC;                             // [TS][dk] (DELTA) or [TS] (SSM)
  float* bs = as + (MODE == MODE_DELTA ? TS * dk : TS); // [TS] beta (DELTA) or dt (SSM)
  const int r = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * VC;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int part = lane % P, col = warp * (32 / P) + lane / P;
  const int j = j0 + col;
  const bool col_ok = j < dv;
  const int q0 = a.cu_q[r], n = a.cu_q[r + 1] - q0;
  const int hq = h / (a.H / a.Hqk);                     // the q/k head (or group) this head reads
  float* S = a.state + (((size_t)a.slots[r] * a.H + h) * dk) * dv;
  float s[REC_RPT];
#pragma unroll
  for (int u = 0; u < REC_RPT; ++u) {
    const int i = part + P * u;
    s[u] = (col_ok && i < dk) ? S[(size_t)i * dv + j] : 0.f;
  }
  const T* qp = (const T*)a.q; const T* kp = (const T*)a.k; const T* vp = (const T*)a.v;
  float head_decay = 1.f, neg_a = 0.f, dt_b = 0.f, d_skip = 0.f;
  if (MODE == MODE_DECAY) head_decay = ((const float*)a.decay)[h];
  if (MODE == MODE_SSM) {
    neg_a = -expf(load_w(a.a_log, a.par_dtype, h));
    dt_b = load_w(a.dt_bias, a.par_dtype, h);
    d_skip = load_w(a.d_skip, a.par_dtype, h);
  }
  if (MODE == MODE_DELTA) neg_a = -expf(load_w(a.a_log, a.par_dtype, h));

  for (int t0 = 0; t0 < n; t0 += TS) {
    const int nt = min(TS, n - t0);
    __syncthreads();                                    // the chunk before has been consumed
    for (int w = tid; w < nt * dk; w += REC_THREADS) {
      const int tt = w / dk, i = w - tt * dk;
      const size_t row = (size_t)(q0 + t0 + tt);
      float qv = to_float(qp[row * a.q_stride + (size_t)hq * dk + i]);
      float kv = to_float(kp[row * a.k_stride + (size_t)hq * dk + i]);
      if (MODE == MODE_DECAY) { qv = silu_f(qv); kv = silu_f(kv); }
      qs[w] = qv;
      ks[w] = kv;
      if (MODE == MODE_DELTA) {
        const float rate = to_float(((const T*)a.rate)[row * a.rate_stride + (size_t)h * dk + i]) +
                           load_w(a.dt_bias, a.par_dtype, (size_t)h * dk + i);
        as[w] = expf(neg_a * softplus_f(rate));
      }
    }
    for (int w = tid; w < nt * VC; w += REC_THREADS) {
      const int tt = w / VC, c = w - tt * VC;
      float vv = 0.f;
      if (j0 + c < dv) vv = to_float(vp[(size_t)(q0 + t0 + tt) * a.v_stride + (size_t)h * dv + j0 + c]);
      if (MODE == MODE_DECAY) vv = silu_f(vv);
      vs[w] = vv;
    }
    if (MODE != MODE_DECAY) {
      for (int tt = tid; tt < nt; tt += REC_THREADS) {
        const float raw = to_float(((const T*)a.aux)[(size_t)(q0 + t0 + tt) * a.aux_stride + h]);
        if (MODE == MODE_SSM) {
          const float dt = softplus_f(raw + dt_b);
          bs[tt] = dt;
          as[tt] = expf(neg_a * dt);
        } else {
          bs[tt] = sigmoid_f(raw);
        }
      }
    }
    __syncthreads();
    if (MODE == MODE_DELTA) {
      // queries and keys become unit vectors (the query also times q_scale): a warp per token and vector
      for (int w = warp; w < 2 * nt; w += REC_WARPS) {
        float* vec = (w < nt ? qs : ks) + (size_t)(w < nt ? w : w - nt) * dk;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) ss += vec[i] * vec[i];
        ss = warp_sum(ss);
        const float f = (w < nt ? a.q_scale : 1.f) / sqrtf(ss + 1e-6f);
        for (int i = lane; i < dk; i += 32) vec[i] *= f;
      }
      __syncthreads();
    }
    for (int tt = 0; tt < nt; ++tt) {
      const float* qt = qs + tt * dk;
      const float* kt = ks + tt * dk;
      const float vv = vs[tt * VC + col];
      float dec = head_decay, u = vv;
      if (MODE == MODE_SSM) { dec = as[tt]; u = bs[tt] * vv; }
      if (MODE == MODE_DELTA) {
        float dot = 0.f;
#pragma unroll
        for (int x = 0; x < REC_RPT; ++x) {
          const int i = part + P * x;
          if (i < dk) {
            s[x] *= as[tt * dk + i];
            dot += s[x] * kt[i];
          }
        }
        for (int o = P >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        u = bs[tt] * (vv - dot);
      }
      float o_acc = 0.f;
#pragma unroll
      for (int x = 0; x < REC_RPT; ++x) {
        const int i = part + P * x;
        if (i < dk) {
          if (MODE != MODE_DELTA) s[x] *= dec;
          s[x] += kt[i] * u;
          o_acc += s[x] * qt[i];
        }
      }
      for (int o = P >> 1; o > 0; o >>= 1) o_acc += __shfl_xor_sync(0xffffffffu, o_acc, o);
      if (MODE == MODE_SSM) o_acc += d_skip * vv;
      if (part == 0 && col_ok) a.out[(size_t)(q0 + t0 + tt) * a.out_stride + (size_t)h * dv + j] = o_acc;
    }
  }
#pragma unroll
  for (int u = 0; u < REC_RPT; ++u) {
    const int i = part + P * u;
    if (col_ok && i < dk) S[(size_t)i * dv + j] = s[u];
  }
}

template <typename T, int MODE>
int launch_recurrence(RecArgs a, int n_rows, cudaStream_t stream) {
  int P = 1;
  while (P * REC_RPT < a.dk) P <<= 1;
  if (P > 32) return SB_ERR_LIMIT;
  a.P = P;
  const int VC = REC_THREADS / P;
  const int per_token = 2 * a.dk + VC + (MODE == MODE_DELTA ? a.dk : 1) + 1;
  int ts = (40 * 1024 / 4) / per_token;
  if (ts > 16) ts = 16;
  if (ts < 1) return SB_ERR_LIMIT;
  a.ts = ts;
  const size_t smem = (size_t)ts * per_token * sizeof(float);
  dim3 grid((a.dv + VC - 1) / VC, a.H, n_rows);
  recurrence_kernel<T, MODE><<<grid, REC_THREADS, smem, stream>>>(a);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------ norm and gate
// out[t, c] = scale * post( rms_g( pre(y[t, c]) ) * w[c mod w_size] ), a warp per (token, group):
// (y is float, or of the activations' type)
//   pre:  times act(gate[t, c']) if the gate comes first; rms_g: divided by the root mean square of the group's
//   values (+ eps inside the root; no division with groups == 0, where a group is just a warp's share of the row);
//   post: times act(gate[t, c']) if the gate comes last. c' = c, or c / (C / gate_cols) for a gate per head.
template <typename T>
__global__ void __launch_bounds__(128) gated_norm_kernel(const void* __restrict__ y, int y_dtype, int y_stride, const T* __restrict__ gate,
                                                         int gate_stride, int gate_cols, int gate_act, int gate_first,
                                                         const void* __restrict__ weight, int w_dtype, int w_size, T* __restrict__ out,
                                                         int out_stride, int n_tokens, int C, int groups, int normalise, float eps,
                                                         float scale) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (wid >= (long long)n_tokens * groups) return;
  const int t = (int)(wid / groups), g = (int)(wid - (long long)t * groups);
  const int gs = C / groups, c0 = g * gs;
  const int per_gate = gate ? C / gate_cols : 1;
  const size_t yr = (size_t)t * y_stride;
  const T* gr = gate ? gate + (size_t)t * gate_stride : nullptr;
  auto gate_of = [&](int c) {
    const float z = to_float(gr[c / per_gate]);
    return gate_act == 1 ? silu_f(z) : sigmoid_f(z);
  };
  float inv = 1.f;
  if (normalise) {
    float ss = 0.f;
    for (int c = c0 + lane; c < c0 + gs; c += 32) {
      float v = load_w(y, y_dtype, yr + c);
      if (gr && gate_first) v *= gate_of(c);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)gs + eps);
  }
  for (int c = c0 + lane; c < c0 + gs; c += 32) {
    float v = load_w(y, y_dtype, yr + c);
    if (gr && gate_first) v *= gate_of(c);
    v *= inv;
    if (weight) v *= load_w(weight, w_dtype, c % w_size);
    if (gr && !gate_first) v *= gate_of(c);
    out[(size_t)t * out_stride + c] = from_float<T>(v * scale);
  }
}

// ------------------------------------------------------------------------------------------ cache write, values normalised
// Keys and values of a step go to their pages, unrotated; with norm_dim > 0 every value head is first divided by
// the root mean square of its first norm_dim elements (what lies beyond them is padding and stays as it is).
// A warp per (token, kv head). Row layout of qkv: H query heads, Hkv key heads, Hkv value heads, D apart.
template <typename T>
__global__ void __launch_bounds__(128) kv_norm_cache_write_kernel(const T* __restrict__ qkv, int stride, const int* __restrict__ positions,
                                                                  const int* __restrict__ token_row, int H, int Hkv, int D, int norm_dim,
                                                                  float eps, T* __restrict__ kc, T* __restrict__ vc,
                                                                  const int* __restrict__ block_table, int bt_width, int ps, int num_pages,
                                                                  int n_tokens, int* __restrict__ errors) {
  const int lane = threadIdx.x & 31;
  const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (wid >= (long long)n_tokens * Hkv) return;
  const int t = (int)(wid / Hkv), hk = (int)(wid - (long long)t * Hkv);
  const int pos = positions[t], blk = pos / ps;
  const int page = (blk < bt_width && pos >= 0) ? block_table[(size_t)token_row[t] * bt_width + blk] : -1;
  if (page < 0 || page >= num_pages) {
    if (lane == 0) atomicAdd(errors, 1);
    return;
  }
  const T* krow = qkv + (size_t)t * stride + (size_t)(H + hk) * D;
  const T* vrow = qkv + (size_t)t * stride + (size_t)(H + Hkv + hk) * D;
  const size_t dst = (((size_t)page * Hkv + hk) * ps + (pos - blk * ps)) * D;
  float inv = 1.f;
  if (norm_dim > 0) {
    float ss = 0.f;
    for (int d = lane; d < norm_dim; d += 32) {
      const float v = to_float(vrow[d]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)norm_dim + eps);
  }
  for (int d = lane; d < D; d += 32) {
    kc[dst + d] = krow[d];
    vc[dst + d] = from_float<T>(to_float(vrow[d]) * inv);
  }
}

}  // namespace

// x [T, C] (row stride x_stride), w [C, taps], bias [C] or null, state float [slots, taps - 1, C], out [T, C].
// act: 0 none, 1 silu. residual: the input itself is added before the activation. A step in which every row brings one
// token (pure_decode) moves the state in the same launch; otherwise a second launch does, after every read.
SB_EXPORT int sb_causal_conv(const void* x, int x_stride, const void* w, const void* bias, float* state, const int* slots,
                             const int* cu_q, const int* token_row, void* out, int out_stride, int C, int taps, int act, int residual,
                             int n_tokens, int n_rows, int pure_decode, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS || n_rows <= 0 || n_rows > 65535 || n_tokens > 65535 * 32) return SB_ERR_LIMIT;
  if (x == out) return SB_ERR_SHAPE;
  dim3 grid((C + CONV_THREADS - 1) / CONV_THREADS, n_tokens), sgrid(grid.x, n_rows);
  if (grid.y > 65535) return SB_ERR_LIMIT;
  if (dtype == SB_DTYPE_F32) {
    causal_conv_kernel<float><<<grid, CONV_THREADS, 0, stream>>>((const float*)x, x_stride, (const float*)w, (const float*)bias, state,
                                                                  slots, cu_q, token_row, (float*)out, out_stride, C, taps, act, residual,
                                                                  pure_decode);
    SB_LAUNCH_CHECK();
    if (!pure_decode && taps > 1)
      conv_state_kernel<float><<<sgrid, CONV_THREADS, 0, stream>>>((const float*)x, x_stride, state, slots, cu_q, C, taps);
  } else if (dtype == SB_DTYPE_BF16) {
    typedef __nv_bfloat16 B;
    causal_conv_kernel<B><<<grid, CONV_THREADS, 0, stream>>>((const B*)x, x_stride, (const B*)w, (const B*)bias, state, slots, cu_q,
                                                              token_row, (B*)out, out_stride, C, taps, act, residual, pure_decode);
    SB_LAUNCH_CHECK();
    if (!pure_decode && taps > 1)
      conv_state_kernel<B><<<sgrid, CONV_THREADS, 0, stream>>>((const B*)x, x_stride, state, slots, cu_q, C, taps);
  } else {
    return SB_ERR_DTYPE;
  }
  SB_LAUNCH_CHECK();
  return 0;
}

// The three recurrences (mode 0: fixed decay per head with silu on q, k, v; 1: selective state space; 2: gated delta
// rule). See RecArgs for what each pointer is; unused ones are null. out is float [T, H * dv].
SB_EXPORT int sb_linear_recurrence(int mode, const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                                   const void* aux, int aux_stride, const void* rate, int rate_stride, const float* decay,
                                   const void* a_log, const void* dt_bias, const void* d_skip, int par_dtype, float* state,
                                   const int* slots, const int* cu_q, float* out, int out_stride, int H, int Hqk, int dk, int dv,
                                   float q_scale, int n_rows, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (H <= 0 || Hqk <= 0 || H % Hqk || dk <= 0 || dv <= 0) return SB_ERR_SHAPE;
  if (n_rows > 65535 || H > 65535 || dk > 32 * REC_RPT) return SB_ERR_LIMIT;
  RecArgs a;
  a.q = q; a.k = k; a.v = v; a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.aux = aux; a.aux_stride = aux_stride; a.rate = rate; a.rate_stride = rate_stride; a.decay = decay;
  a.a_log = a_log; a.dt_bias = dt_bias; a.d_skip = d_skip; a.par_dtype = par_dtype; a.state = state; a.slots = slots; a.cu_q = cu_q;
  a.out = out; a.out_stride = out_stride; a.H = H; a.Hqk = Hqk; a.dk = dk; a.dv = dv; a.P = 1; a.ts = 1; a.q_scale = q_scale;
  if (dtype == SB_DTYPE_F32) {
    if (mode == MODE_DECAY) return launch_recurrence<float, MODE_DECAY>(a, n_rows, stream);
    if (mode == MODE_SSM) return launch_recurrence<float, MODE_SSM>(a, n_rows, stream);
    if (mode == MODE_DELTA) return launch_recurrence<float, MODE_DELTA>(a, n_rows, stream);
  } else if (dtype == SB_DTYPE_BF16) {
    if (mode == MODE_DECAY) return launch_recurrence<__nv_bfloat16, MODE_DECAY>(a, n_rows, stream);
    if (mode == MODE_SSM) return launch_recurrence<__nv_bfloat16, MODE_SSM>(a, n_rows, stream);
    if (mode == MODE_DELTA) return launch_recurrence<__nv_bfloat16, MODE_DELTA>(a, n_rows, stream);
  } else {
    return SB_ERR_DTYPE;
  }
  return SB_ERR_SHAPE;
}

// y [T, C], float or the activations' type (y_dtype); gate [T, gate_cols] or null (gate_act 0 sigmoid, 1 silu; gate_first: before the norm); weight [w_size]
// or null (w_size divides C); groups > 0: each of the groups equal parts of a row is divided by its own root mean square.
SB_EXPORT int sb_gated_norm(const void* y, int y_dtype, int y_stride, const void* gate, int gate_stride, int gate_cols, int gate_act, int gate_first,
                            const void* weight, int w_dtype, int w_size, void* out, int out_stride, int n_tokens, int C, int groups,
                            float eps, float scale, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0 || C <= 0) return 0;
  const int normalise = groups > 0 ? 1 : 0;
  if (groups <= 0) groups = gate ? gate_cols : 1;
  if (C % groups || (gate && (gate_cols <= 0 || C % gate_cols)) || (weight && (w_size <= 0 || C % w_size))) return SB_ERR_SHAPE;
  const long long warps = (long long)n_tokens * groups;
  const long long blocks = (warps + 3) / 4;
  if (blocks > 0x7fffffffLL) return SB_ERR_LIMIT;
  if (dtype == SB_DTYPE_F32)
    gated_norm_kernel<float><<<(unsigned)blocks, 128, 0, stream>>>(y, y_dtype, y_stride, (const float*)gate, gate_stride, gate_cols, gate_act,
                                                                    gate_first, weight, w_dtype, w_size, (float*)out, out_stride, n_tokens,
                                                                    C, groups, normalise, eps, scale);
  else if (dtype == SB_DTYPE_BF16)
    gated_norm_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, stream>>>(y, y_dtype, y_stride, (const __nv_bfloat16*)gate, gate_stride, gate_cols,
                                                                            gate_act, gate_first, weight, w_dtype, w_size,
                                                                            (__nv_bfloat16*)out, out_stride, n_tokens, C, groups, normalise,
                                                                            eps, scale);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}

SB_EXPORT int sb_kv_norm_cache_write(const void* qkv, int stride, const int* positions, const int* token_row, int H, int Hkv, int D,
                                     int norm_dim, float eps, void* kc, void* vc, const int* block_table, int bt_width, int ps,
                                     int num_pages, int n_tokens, int* errors, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H < 0 || Hkv <= 0 || D <= 0 || norm_dim < 0 || norm_dim > D || ps <= 0 || bt_width <= 0) return SB_ERR_SHAPE;
  const long long blocks = ((long long)n_tokens * Hkv + 3) / 4;
  if (blocks > 0x7fffffffLL) return SB_ERR_LIMIT;
  if (dtype == SB_DTYPE_F32)
    kv_norm_cache_write_kernel<float><<<(unsigned)blocks, 128, 0, stream>>>((const float*)qkv, stride, positions, token_row, H, Hkv, D,
                                                                             norm_dim, eps, (float*)kc, (float*)vc, block_table, bt_width,
                                                                             ps, num_pages, n_tokens, errors);
  else if (dtype == SB_DTYPE_BF16)
    kv_norm_cache_write_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, stream>>>(
        (const __nv_bfloat16*)qkv, stride, positions, token_row, H, Hkv, D, norm_dim, eps, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc,
        block_table, bt_width, ps, num_pages, n_tokens, errors);
  else
    return SB_ERR_DTYPE;
  SB_LAUNCH_CHECK();
  return 0;
}
