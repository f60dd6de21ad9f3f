// The gated delta rule: a matrix state S [dk, dv] per request and head that every token first decays as a whole,
// then corrects so that reading it with the token's key gives (a step towards) the token's value, then reads:
//
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
//
// Unlike a recurrence that only adds outer products, the write depends on the state (S^T k), so no token can be
// walked before its predecessor is done.  Everything here is 32-bit: the convolution's sums, activations, unit
// norms, gates, decays, the state and its sums.  The kernels:
//
//   conv_unit_prep   from projected rows (split-K partials are added on the way): a short causal convolution per
//                    channel over a request's time axis (the last taps - 1 inputs of a request are its state), an
//                    activation, then q and k made unit vectors per head (q scaled), beta = sigmoid(b) and the decay
//                    g = exp(-rate * softplus(a + bias)) per head.
//   delta_scan       the recurrence over each request's tokens, in order; the state lives in registers.
//
// Every sum runs in an order that depends on the token alone, so a token's result does not change with the batch or
// with how its prompt was cut into steps.
#include "common.cuh"

// Projected rows that may still be split-K partials: element (row, col) = sum_z p[z * split_stride + row * ld + col].
struct RowsView {
  const float* p;
  long long split_stride;
  long long ld;
  int splits;
  int pad_;
};

__device__ __forceinline__ float rows_at(const RowsView& v, size_t row, int col) {
  float s = 0.f;
  for (int z = 0; z < v.splits; ++z) s += v.p[(size_t)z * v.split_stride + row * v.ld + col];
  return s;
}

#define DELTA_MAX_TAPS 16
enum { DELTA_ACT_NONE = 0, DELTA_ACT_SILU = 1 };

__device__ __forceinline__ float delta_act(float x, int act) { return act == DELTA_ACT_SILU ? x / (1.f + expf(-x)) : x; }

struct PrepParams {
  RowsView proj;            // columns: [q: G dk | k: G dk | v: H dv] from column 0 (the convolved channels, C of them),
  int b_col, a_col;         // beta's and the decay's logits, H columns each
  const float* conv_w;      // [C, taps], the last column is the current token's
  float* conv_state;        // [slots, taps - 1, C]: a request's last inputs, oldest first (zeros before its start)
  const float* rate_log;    // [H]: the decay's rate is exp(rate_log)
  const float* a_bias;      // [H]
  const int* cu_q;
  const int* q_start;
  const int* slot_ids;
  const int* req_of_token;
  const int* positions;
  float* qo;                // [N, G, dk] unit vectors times q_scale
  float* ko;                // [N, G, dk] unit vectors
  float* vo;                // [N, H, dv]
  float* beta;              // [N, H]
  float* decay;             // [N, H]
  int N, R, G, H, dk, dv, taps, act;
  float unit_eps, q_scale;
};

// The convolved and activated value of channel c at token row n.  `first` = the row of the request's first token in
// this step; taps that reach before it come from `old` (the state as it was before the step, taps - 1 entries).
__device__ __forceinline__ float conv_at(const PrepParams& P, size_t n, int first, int c, const float* old) {
  float acc = 0.f;
  for (int j = 0; j < P.taps; ++j) {
    const long long s = (long long)n - P.taps + 1 + j;
    const float x = s >= first ? rows_at(P.proj, (size_t)s, c) : old[s - first + P.taps - 1];
    acc = fmaf(P.conv_w[(size_t)c * P.taps + j], x, acc);
  }
  return delta_act(acc, P.act);
}

// One head group (q or k head of dk channels, or v head of dv) of one token by one warp.
__device__ __forceinline__ void prep_group(const PrepParams& P, size_t n, int first, int grp, const float* state_old, float* old_buf) {
  const int lane = threadIdx.x & 31;
  const int C_qk = P.G * P.dk;
  const bool is_q = grp < P.G, is_k = !is_q && grp < 2 * P.G;
  const int size = (is_q || is_k) ? P.dk : P.dv;
  const int c0 = is_q ? grp * P.dk : (is_k ? C_qk + (grp - P.G) * P.dk : 2 * C_qk + (grp - 2 * P.G) * P.dv);
  const int C = 2 * C_qk + P.H * P.dv;
  float* dst = is_q ? P.qo + (n * P.G + grp) * P.dk
                    : (is_k ? P.ko + (n * P.G + (grp - P.G)) * P.dk : P.vo + (n * P.H + (grp - 2 * P.G)) * P.dv);
  float ss = 0.f;
  for (int i = lane; i < size; i += 32) {
    if (state_old)
      for (int t = 0; t < P.taps - 1; ++t) old_buf[t] = state_old[(size_t)t * C + c0 + i];
    const float y = conv_at(P, n, first, c0 + i, old_buf);
    dst[i] = y;
    ss = fmaf(y, y, ss);
  }
  if (is_q || is_k) {
    ss = warp_sum(ss);
    const float inv = (is_q ? P.q_scale : 1.f) / sqrtf(ss + P.unit_eps);
    __syncwarp();
    for (int i = lane; i < size; i += 32) dst[i] *= inv;  // each lane scales what it wrote itself
  }
}

__device__ __forceinline__ void prep_gates(const PrepParams& P, size_t n) {
  for (int h = threadIdx.x; h < P.H; h += blockDim.x) {
    const float b = rows_at(P.proj, n, P.b_col + h);
    P.beta[n * P.H + h] = 1.f / (1.f + expf(-b));
    const float a = rows_at(P.proj, n, P.a_col + h) + P.a_bias[h];
    const float sp = fmaxf(a, 0.f) + log1pf(expf(-fabsf(a)));  // softplus
    P.decay[n * P.H + h] = expf(-expf(P.rate_log[h]) * sp);
  }
}

// Blocks [0, N): one token each, unless it is among the first taps - 1 of its request's portion: those need the
// state, and block N + r serves them for request r and then moves the state on; no other block touches the state.
__global__ void __launch_bounds__(256) conv_unit_prep_kernel(const PrepParams P) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int groups = 2 * P.G + P.H;
  const int C = 2 * P.G * P.dk + P.H * P.dv;
  float old[DELTA_MAX_TAPS];
  const int b = blockIdx.x;
  if (b < P.N) {
    const int r = P.req_of_token[b];
    if (P.positions[b] - P.q_start[r] < P.taps - 1) return;
    for (int g = warp; g < groups; g += nwarp) prep_group(P, b, 0, g, nullptr, old);  // never reaches before the portion
    prep_gates(P, b);
    return;
  }
  const int r = b - P.N;
  const int n0 = P.cu_q[r], qlen = P.cu_q[r + 1] - n0;
  float* st = P.conv_state + (size_t)P.slot_ids[r] * (P.taps - 1) * C;
  const int head = qlen < P.taps - 1 ? qlen : P.taps - 1;
  for (int i = 0; i < head; ++i) {
    for (int g = warp; g < groups; g += nwarp) prep_group(P, (size_t)n0 + i, n0, g, st, old);
    prep_gates(P, (size_t)n0 + i);
  }
  __syncthreads();  // every read of the old state is done
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    for (int t = 0; t < P.taps - 1; ++t) old[t] = st[(size_t)t * C + c];
    for (int t = 0; t < P.taps - 1; ++t) {
      const int s = qlen - (P.taps - 1) + t;
      st[(size_t)t * C + c] = s >= 0 ? rows_at(P.proj, (size_t)n0 + s, c) : old[s + P.taps - 1];
    }
  }
}

JLX_API int jlx_conv_unit_prep(const RowsView* proj, int b_col, int a_col, const float* conv_w, float* conv_state,
                               const float* rate_log, const float* a_bias, const int* cu_q, const int* q_start,
                               const int* slot_ids, const int* req_of_token, const int* positions, float* qo, float* ko,
                               float* vo, float* beta, float* decay, int N, int R, int G, int H, int dk, int dv, int taps,
                               int act, float unit_eps, float q_scale, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && R >= 0 && G > 0 && H > 0 && dk > 0 && dv > 0, "conv_unit_prep: bad sizes N=%d R=%d G=%d H=%d dk=%d dv=%d", N, R, G,
              H, dk, dv);
  JLX_REQUIRE(H % G == 0, "conv_unit_prep: %d heads are no multiple of %d key heads", H, G);
  JLX_REQUIRE(taps >= 1 && taps <= DELTA_MAX_TAPS, "conv_unit_prep: %d taps; supported 1..%d", taps, DELTA_MAX_TAPS);
  JLX_REQUIRE(taps == 1 || conv_state, "conv_unit_prep: a convolution over more than one tap needs its state");
  JLX_REQUIRE(act == DELTA_ACT_NONE || act == DELTA_ACT_SILU, "conv_unit_prep: unknown activation %d", act);
  if (N == 0) return 0;
  PrepParams P;
  P.proj = *proj; P.b_col = b_col; P.a_col = a_col; P.conv_w = conv_w; P.conv_state = conv_state; P.rate_log = rate_log;
  P.a_bias = a_bias; P.cu_q = cu_q; P.q_start = q_start; P.slot_ids = slot_ids; P.req_of_token = req_of_token;
  P.positions = positions; P.qo = qo; P.ko = ko; P.vo = vo; P.beta = beta; P.decay = decay;
  P.N = N; P.R = R; P.G = G; P.H = H; P.dk = dk; P.dv = dv; P.taps = taps; P.act = act; P.unit_eps = unit_eps; P.q_scale = q_scale;
  const int groups = 2 * G + H;
  const int warps = groups < 8 ? groups : 8;
  JLX_CUDA(jlx_launch_pdl(conv_unit_prep_kernel, dim3(N + (taps > 1 ? R : 0)), dim3(warps * 32), 0, stream, P));
  JLX_LAUNCH_CHECK("conv_unit_prep");
  return 0;
}

// ------------------------------------------------------------------------------------------------ the recurrence
// One block per (request, head, slice of COLS value columns).  A column of S belongs to four neighbouring lanes, each
// keeping RPT of its rows in registers (row i = part * RPT + r; rows from dk on hold zeros and stay zero), so the two
// sums over a column's rows are RPT products per lane and two shuffles; no barrier stands between two tokens.  Both
// sums are taken over the state as the token found it:
//
//     a = k . S[:, j],  b = q . S[:, j];   u = beta (v_j - g a);   S[:, j] <- g S[:, j] + k u;   o_j = g b + (q . k) u,
//
// which is the rule above with the read-out written through the update (o = (g S + k u^T)^T q), so that a token costs
// one round of shuffles.  The tokens' q and k rows, v slice, beta, g and q . k come through shared memory SCAN_TB
// tokens at a time.  A token's arithmetic is the same wherever it stands in a step.
#define SCAN_TB 16
#define DELTA_COLS 32  // value columns per block: 128 threads

template <int RPT>
__global__ void __launch_bounds__(128) delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                         const float* __restrict__ v, const float* __restrict__ beta,
                                                         const float* __restrict__ decay, float* __restrict__ state,
                                                         const int* __restrict__ cu_q, const int* __restrict__ slot_ids,
                                                         float* __restrict__ o, int G, int H, int dk, int dv) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  constexpr int LDP = RPT + 4;       // a part's rows in shared memory, padded so that the four parts fall into other banks
  constexpr int ROW = 4 * LDP;
  __shared__ __align__(16) float qs[SCAN_TB][ROW], ks[SCAN_TB][ROW];
  __shared__ float vs[SCAN_TB][DELTA_COLS], bs[SCAN_TB], gs[SCAN_TB], qk[SCAN_TB];
  const int r = blockIdx.z, hd = blockIdx.y, j0 = blockIdx.x * DELTA_COLS;
  const int kh = hd / (H / G);
  const int part = threadIdx.x & 3, col = threadIdx.x >> 2;
  const int j = j0 + col;
  const bool col_ok = j < dv;
  pdl_wait();
  const int n0 = cu_q[r], n1 = cu_q[r + 1];
  if (n1 <= n0) return;
  float* S = state + ((size_t)slot_ids[r] * H + hd) * dk * dv;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int row = part * RPT + i;
    s[i] = (col_ok && row < dk) ? S[(size_t)row * dv + j] : 0.f;
  }
  for (int t0 = n0; t0 < n1; t0 += SCAN_TB) {
    const int cnt = min(SCAN_TB, n1 - t0);
    __syncthreads();  // the previous group is walked
    for (int idx = threadIdx.x; idx < cnt * 4 * RPT; idx += 128) {
      const int t = idx / (4 * RPT), e = idx - t * 4 * RPT;  // e = the row
      const int at = (e / RPT) * LDP + e % RPT;
      const size_t src = ((size_t)(t0 + t) * G + kh) * dk + e;
      qs[t][at] = e < dk ? q[src] : 0.f;
      ks[t][at] = e < dk ? k[src] : 0.f;
    }
    for (int idx = threadIdx.x; idx < cnt * DELTA_COLS; idx += 128) {
      const int t = idx / DELTA_COLS, c = idx - t * DELTA_COLS;
      vs[t][c] = j0 + c < dv ? v[((size_t)(t0 + t) * H + hd) * dv + j0 + c] : 0.f;
    }
    if ((int)threadIdx.x < cnt) {
      bs[threadIdx.x] = beta[(size_t)(t0 + threadIdx.x) * H + hd];
      gs[threadIdx.x] = decay[(size_t)(t0 + threadIdx.x) * H + hd];
    }
    __syncthreads();
    // q . k of every token of the group: eight threads per token, rows in a fixed order (the padding between the
    // parts is never written, so the product walks rows, not entries)
    {
      const int t = threadIdx.x >> 3, sub = threadIdx.x & 7;
      float d = 0.f;
      if (t < cnt)
        for (int e = sub; e < 4 * RPT; e += 8) {
          const int at = (e / RPT) * LDP + e % RPT;
          d = fmaf(qs[t][at], ks[t][at], d);
        }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      if (t < cnt && sub == 0) qk[t] = d;
    }
    __syncthreads();
    for (int t = 0; t < cnt; ++t) {
      const float* kp = &ks[t][part * LDP];
      const float* qp = &qs[t][part * LDP];
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kp + i);
        const float4 q4 = *reinterpret_cast<const float4*>(qp + i);
        a0 = fmaf(k4.x, s[i], a0); a1 = fmaf(k4.y, s[i + 1], a1); a0 = fmaf(k4.z, s[i + 2], a0); a1 = fmaf(k4.w, s[i + 3], a1);
        b0 = fmaf(q4.x, s[i], b0); b1 = fmaf(q4.y, s[i + 1], b1); b0 = fmaf(q4.z, s[i + 2], b0); b1 = fmaf(q4.w, s[i + 3], b1);
      }
      float a = a0 + a1, b = b0 + b1;
      a += __shfl_xor_sync(0xffffffffu, a, 1);
      b += __shfl_xor_sync(0xffffffffu, b, 1);
      a += __shfl_xor_sync(0xffffffffu, a, 2);
      b += __shfl_xor_sync(0xffffffffu, b, 2);
      const float g = gs[t];
      const float u = bs[t] * (vs[t][col] - g * a);
#pragma unroll
      for (int i = 0; i < RPT; i += 4) {  // the key's rows once more from shared memory: cheaper than RPT registers
        const float4 k4 = *reinterpret_cast<const float4*>(kp + i);
        s[i] = fmaf(k4.x, u, g * s[i]); s[i + 1] = fmaf(k4.y, u, g * s[i + 1]);
        s[i + 2] = fmaf(k4.z, u, g * s[i + 2]); s[i + 3] = fmaf(k4.w, u, g * s[i + 3]);
      }
      if (part == 0 && col_ok) o[((size_t)(t0 + t) * H + hd) * dv + j] = fmaf(qk[t], u, g * b);
    }
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int row = part * RPT + i;
    if (col_ok && row < dk) S[(size_t)row * dv + j] = s[i];
  }
}

// q, k: float32 [N, G, dk]; v, o: [N, H, dv]; beta, decay: [N, H]; state: float32 [slots, H, dk, dv].
JLX_API int jlx_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* decay, float* state,
                           const int* cu_q, const int* slot_ids, float* o, int R, int G, int H, int dk, int dv, cudaStream_t stream) {
  JLX_REQUIRE(R >= 0 && G > 0 && H > 0 && dk > 0 && dv > 0 && H % G == 0, "delta_scan: bad sizes R=%d G=%d H=%d dk=%d dv=%d", R, G, H, dk, dv);
  JLX_REQUIRE(dk <= 256, "delta_scan: key size %d is above the supported maximum 256", dk);
  JLX_REQUIRE(H <= 65535 && R <= 65535, "delta_scan: too many heads or requests");
  if (R == 0) return 0;
  const dim3 grid((dv + DELTA_COLS - 1) / DELTA_COLS, H, R);
  const int rpt = (dk + 3) / 4;
#define DELTA_LAUNCH(RPT)                                                                                                \
  JLX_CUDA(jlx_launch_pdl(delta_scan_kernel<RPT>, grid, dim3(128), 0, stream, q, k, v, beta, decay, state, cu_q, slot_ids, o, G, H, dk, dv))
  if (rpt <= 4) DELTA_LAUNCH(4);
  else if (rpt <= 8) DELTA_LAUNCH(8);
  else if (rpt <= 16) DELTA_LAUNCH(16);
  else if (rpt <= 24) DELTA_LAUNCH(24);
  else if (rpt <= 32) DELTA_LAUNCH(32);
  else if (rpt <= 48) DELTA_LAUNCH(48);
  else DELTA_LAUNCH(64);
#undef DELTA_LAUNCH
  JLX_LAUNCH_CHECK("delta_scan");
  return 0;
}
