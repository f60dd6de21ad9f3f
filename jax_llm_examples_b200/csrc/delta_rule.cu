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
//   delta_gram       the products between the keys and queries of each group of DELTA_TB tokens, once per key head
//                    (steps that hold prompts).
//   delta_scan       the recurrence over each request's tokens, a group at a time; the state lives in registers.
//
// Nothing of another request enters a token's sums, so a token's result does not change with the batch.  In
// conv_unit_prep the order of a sum depends on the token alone; in delta_scan it also depends on where the token stands
// in its group, and groups count from the request's first token of the step: cutting a prompt elsewhere moves the
// last bits of a result, no more.
#include <type_traits>

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
  int vec;                  // 16-byte accesses are possible (prep_group4)
  int pad_;
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

// The same for sizes and addresses that allow 16-byte accesses (every head size, row length and column offset a
// multiple of four floats): a lane takes four neighbouring channels at a time, so a tap costs one load per split
// instead of four, and heads of up to 256 channels stay in registers between the sum of squares and the store.  A
// channel's sum runs over its taps in the same order as above.
__device__ __forceinline__ float4 rows_at4(const RowsView& v, size_t row, int col) {
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < v.splits; ++z) {
    const float4 x = *reinterpret_cast<const float4*>(v.p + (size_t)z * v.split_stride + row * v.ld + col);
    s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
  }
  return s;
}

__device__ __forceinline__ void prep_group4(const PrepParams& P, size_t n, int first, int grp, const float* old) {
  const int lane = threadIdx.x & 31;
  const int C_qk = P.G * P.dk;
  const bool is_q = grp < P.G, is_k = !is_q && grp < 2 * P.G;
  const int size = (is_q || is_k) ? P.dk : P.dv;
  const int c0 = is_q ? grp * P.dk : (is_k ? C_qk + (grp - P.G) * P.dk : 2 * C_qk + (grp - 2 * P.G) * P.dv);
  const int C = 2 * C_qk + P.H * P.dv;
  float* dst = is_q ? P.qo + (n * P.G + grp) * P.dk
                    : (is_k ? P.ko + (n * P.G + (grp - P.G)) * P.dk : P.vo + (n * P.H + (grp - 2 * P.G)) * P.dv);
  float4 acc[2];
  acc[0] = acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < P.taps; ++j) {
    const long long s = (long long)n - P.taps + 1 + j;
    const bool fresh = s >= first;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int i = lane * 4 + 128 * h;
      if (i < size) {
        const float4 x = fresh ? rows_at4(P.proj, (size_t)s, c0 + i)
                               : *reinterpret_cast<const float4*>(old + (size_t)(s - first + P.taps - 1) * C + c0 + i);
        const float* w = P.conv_w + (size_t)(c0 + i) * P.taps + j;
        acc[h].x = fmaf(w[0], x.x, acc[h].x);
        acc[h].y = fmaf(w[P.taps], x.y, acc[h].y);
        acc[h].z = fmaf(w[2 * P.taps], x.z, acc[h].z);
        acc[h].w = fmaf(w[3 * P.taps], x.w, acc[h].w);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int h = 0; h < 2; ++h)
    if (lane * 4 + 128 * h < size) {
      acc[h].x = delta_act(acc[h].x, P.act); acc[h].y = delta_act(acc[h].y, P.act);
      acc[h].z = delta_act(acc[h].z, P.act); acc[h].w = delta_act(acc[h].w, P.act);
      ss = fmaf(acc[h].x, acc[h].x, ss); ss = fmaf(acc[h].y, acc[h].y, ss);
      ss = fmaf(acc[h].z, acc[h].z, ss); ss = fmaf(acc[h].w, acc[h].w, ss);
    }
  float inv = 1.f;
  if (is_q || is_k) inv = (is_q ? P.q_scale : 1.f) / sqrtf(warp_sum(ss) + P.unit_eps);
#pragma unroll
  for (int h = 0; h < 2; ++h)
    if (lane * 4 + 128 * h < size)
      *reinterpret_cast<float4*>(dst + lane * 4 + 128 * h) = make_float4(acc[h].x * inv, acc[h].y * inv, acc[h].z * inv, acc[h].w * inv);
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
  const bool vec = P.vec != 0;
  if (b < P.N) {
    const int r = P.req_of_token[b];
    if (P.positions[b] - P.q_start[r] < P.taps - 1) return;
    for (int g = warp; g < groups; g += nwarp) {  // never reaches before the portion
      if (vec) prep_group4(P, b, 0, g, nullptr);
      else prep_group(P, b, 0, g, nullptr, old);
    }
    prep_gates(P, b);
    return;
  }
  const int r = b - P.N;
  const int n0 = P.cu_q[r], qlen = P.cu_q[r + 1] - n0;
  float* st = P.conv_state + (size_t)P.slot_ids[r] * (P.taps - 1) * C;
  const int head = qlen < P.taps - 1 ? qlen : P.taps - 1;
  for (int i = 0; i < head; ++i) {
    for (int g = warp; g < groups; g += nwarp) {
      if (vec) prep_group4(P, (size_t)n0 + i, n0, g, st);
      else prep_group(P, (size_t)n0 + i, n0, g, st, old);
    }
    prep_gates(P, (size_t)n0 + i);
  }
  __syncthreads();  // every read of the old state is done
  if (vec && P.taps <= 4) {  // four channels of a thread at a time: all loads, then the stores
    for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
      float4 keep[3];
#pragma unroll
      for (int t = 0; t < 3; ++t)
        if (t < P.taps - 1) {
          const int s = qlen - (P.taps - 1) + t;
          keep[t] = s >= 0 ? rows_at4(P.proj, (size_t)n0 + s, c) : *reinterpret_cast<const float4*>(st + (size_t)(t + qlen) * C + c);
        }
#pragma unroll
      for (int t = 0; t < 3; ++t)
        if (t < P.taps - 1) *reinterpret_cast<float4*>(st + (size_t)t * C + c) = keep[t];
    }
    return;
  }
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
  const auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
  P.vec = dk % 4 == 0 && dv % 4 == 0 && dk <= 256 && dv <= 256 && proj->ld % 4 == 0 && (proj->splits == 1 || proj->split_stride % 4 == 0) &&
          al16(proj->p) && al16(qo) && al16(ko) && al16(vo) && (!conv_state || al16(conv_state));
  P.pad_ = 0;
  const int groups = 2 * G + H;
  const int warps = groups < 8 ? groups : 8;
  JLX_CUDA(jlx_launch_pdl(conv_unit_prep_kernel, dim3(N + (taps > 1 ? R : 0)), dim3(warps * 32), 0, stream, P));
  JLX_LAUNCH_CHECK("conv_unit_prep");
  return 0;
}

// ------------------------------------------------------------------------------------------------ the recurrence
// One block of DELTA_W warps per (request, head, slice of 32 value columns).  Lane = a value column; warp w keeps rows
// [w NR, (w+1) NR) of S for that column in registers (rows from dk on hold zeros and stay zero), so a key's or query's
// rows are read from shared memory at one address by the whole warp.
//
// Walking token by token, every token waits for its predecessor's write (S^T k needs the state just written): one
// long chain of dependent sums per token.  The kernel walks DELTA_TB tokens at a time instead.  With c_t = g_0 ... g_t
// (decays of the group), the state S0 the group found, and column j:
//
//     P_t = k_t . S0[:, j],   B_t = q_t . S0[:, j]                                   (no token waits for another)
//     a_t = c_t P_t + sum_{s<t}  (c_t / c_s) (k_s . k_t) u_s,    u_t = beta_t (v_tj - a_t)
//     o_tj = c_t B_t + sum_{s<=t} (c_t / c_s) (k_s . q_t) u_s                        (scalars only: a short chain)
//     S[:, j] <- c_last S0[:, j] + sum_t (c_last / c_t) k_t u_t                      (no token waits for another)
//
// which is the rule above with the sums taken in another order; nothing is inverted and nothing leaves 32-bit.  The
// ratios c_t / c_s are running products of decays, never quotients: (c_t / c_s) u_s is kept per write and decays with
// every later token, and is what the state gets at the group's end.  The warps' parts of P and B meet in shared
// memory once per group (warp w adds token w's); every warp then walks the scalars (it needs all u for its rows),
// and token t's o is made by warp t.  The products k_s . k_t and k_s . q_t do not depend on the column or on the value head: delta_gram
// makes them once per token and key head for steps that hold prompts; with single tokens only, a block makes its own
// (one product).  Rows, v slice, beta, g and the products come through shared memory, two buffers taking turns:
// while a group is walked, asynchronous copies bring the next.  Groups count from a request's first token of the
// step, so the order of a token's sums, and with it the last bits of its result, depends on where the step begins;
// nothing else in the batch enters.
#define DELTA_TB 8
#define DELTA_W 8  // warps of a scan block: as many as tokens in a group

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// gram [N, G, 2, DELTA_TB]: for token n, the t-th of its group (groups count from its request's first token of the
// step), [0][s] = k_(n-t+s) . q_n for s <= t and [1][s] = k_(n-t+s) . k_n for s < t.  The rest is never read.
// One warp per (token, key head).
__global__ void __launch_bounds__(256) delta_gram_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                         const int* __restrict__ cu_q, const int* __restrict__ req_of_token,
                                                         float* __restrict__ gram, int G, int dk) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int n = blockIdx.x, lane = threadIdx.x & 31;
  const int t = (n - cu_q[req_of_token[n]]) % DELTA_TB;
  for (int kh = threadIdx.x >> 5; kh < G; kh += blockDim.x >> 5) {
    const float* qn = q + ((size_t)n * G + kh) * dk;
    const float* kn = k + ((size_t)n * G + kh) * dk;
    float* out = gram + ((size_t)n * G + kh) * 2 * DELTA_TB;
    for (int s = 0; s <= t; ++s) {
      const float* y = k + ((size_t)(n - t + s) * G + kh) * dk;
      float dq = 0.f, dkk = 0.f;
      for (int i = lane; i < dk; i += 32) {
        dq = fmaf(qn[i], y[i], dq);
        dkk = fmaf(kn[i], y[i], dkk);
      }
      dq = warp_sum(dq);
      dkk = warp_sum(dkk);
      if (lane == 0) {
        out[s] = dq;
        out[DELTA_TB + s] = dkk;
      }
    }
  }
}

template <int NR>
__global__ void __launch_bounds__(DELTA_W * 32) delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                         const float* __restrict__ v, const float* __restrict__ beta,
                                                         const float* __restrict__ decay, float* __restrict__ state,
                                                         const int* __restrict__ cu_q, const int* __restrict__ slot_ids,
                                                         const float* __restrict__ gram, float* __restrict__ o, int G, int H,
                                                         int dk, int dv) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  constexpr int T = DELTA_TB;
  constexpr int W = DELTA_W;
  static_assert(T % 4 == 0 && NR % 4 == 0 && W == T, "rows and products are read four at a time; a warp per token of a group");
  extern __shared__ __align__(16) float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int dkp = W * NR;
  constexpr int stage_floats = 2 * T * dkp + T * 32 + 2 * T + 2 * T * T;  // q rows | k rows | v slice | beta | g | k.q | k.k
  float* parts = smem + 2 * stage_floats;                                   // [2][T][W][32]: the warps' parts of P and B
  float* sums = parts + 2 * T * W * 32;                                     // [2][T][32]: P and B
  const int r = blockIdx.z, hd = blockIdx.y, j0 = blockIdx.x * 32;
  const int kh = hd / (H / G);
  const int j = j0 + lane;
  const bool col_ok = j < dv;
  const int i0 = warp * NR;
  if (dk < dkp || dv - j0 < 32) {  // what no copy ever writes: rows beyond dk, columns beyond dv
    for (int idx = threadIdx.x; idx < 2 * stage_floats; idx += blockDim.x) smem[idx] = 0.f;
    __syncthreads();
  }
  pdl_wait();
  const int n0 = cu_q[r], n1 = cu_q[r + 1];
  if (n1 <= n0) return;
  float* S = state + ((size_t)slot_ids[r] * H + hd) * dk * dv;
  float s[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) s[i] = (col_ok && i0 + i < dk) ? S[(size_t)(i0 + i) * dv + j] : 0.f;
  const bool vec = (dk & 3) == 0 && (dv & 3) == 0 && ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0);
  const int nv = min(32, dv - j0);
  auto stage = [&](int t0, int b) {  // asynchronous copies of a group's rows into buffer b
    float* st = smem + b * stage_floats;
    const int cnt = min(T, n1 - t0);
    if (vec) {
      const int dk4 = dk >> 2, nv4 = nv >> 2;
      for (int idx = threadIdx.x; idx < cnt * dk4; idx += blockDim.x) {
        const int tt = idx / dk4, e = (idx - tt * dk4) << 2;
        const size_t src = ((size_t)(t0 + tt) * G + kh) * dk + e;
        cp_async16(st + tt * dkp + e, q + src);
        cp_async16(st + T * dkp + tt * dkp + e, k + src);
      }
      for (int idx = threadIdx.x; idx < cnt * nv4; idx += blockDim.x) {
        const int tt = idx / nv4, l = (idx - tt * nv4) << 2;
        cp_async16(st + 2 * T * dkp + tt * 32 + l, v + ((size_t)(t0 + tt) * H + hd) * dv + j0 + l);
      }
    } else {
      for (int idx = threadIdx.x; idx < cnt * dk; idx += blockDim.x) {
        const int tt = idx / dk, e = idx - tt * dk;
        const size_t src = ((size_t)(t0 + tt) * G + kh) * dk + e;
        cp_async4(st + tt * dkp + e, q + src);
        cp_async4(st + T * dkp + tt * dkp + e, k + src);
      }
      for (int idx = threadIdx.x; idx < cnt * nv; idx += blockDim.x) {
        const int tt = idx / nv, l = idx - tt * nv;
        cp_async4(st + 2 * T * dkp + tt * 32 + l, v + ((size_t)(t0 + tt) * H + hd) * dv + j0 + l);
      }
    }
    float* small = st + 2 * T * dkp + T * 32;
    for (int idx = threadIdx.x; idx < cnt; idx += blockDim.x) {
      cp_async4(small + idx, beta + (size_t)(t0 + idx) * H + hd);
      cp_async4(small + T + idx, decay + (size_t)(t0 + idx) * H + hd);
    }
    if (gram)  // a token's 2 T products are 16-byte aligned rows
      for (int idx = threadIdx.x; idx < cnt * (2 * T / 4); idx += blockDim.x) {
        const int tt = idx / (2 * T / 4), part = idx - tt * (2 * T / 4);  // part: T / 4 pieces of k.q, then of k.k
        const int which = part / (T / 4), piece = part - which * (T / 4);
        cp_async16(small + 2 * T + which * T * T + tt * T + piece * 4,
                   gram + (((size_t)(t0 + tt) * G + kh) * 2 + which) * T + piece * 4);
      }
    cp_async_commit();
  };

  stage(n0, 0);
  int b = 0;
  for (int t0 = n0; t0 < n1; t0 += T, b ^= 1) {
    const int cnt = min(T, n1 - t0);
    cp_async_wait_all();
    __syncthreads();  // this group's rows are there; the group before is walked: its buffer and the parts are free
    if (t0 + T < n1) stage(t0 + T, b ^ 1);
    float* st = smem + b * stage_floats;
    const float* qs = st;
    const float* ks = qs + T * dkp;
    const float* vs = ks + T * dkp;
    const float* bs = vs + T * 32;
    const float* gs = bs + T;
    float* Mqk = st + 2 * T * dkp + T * 32 + 2 * T;  // [T][T], s <= t: k_s . q_t
    float* Mkk = Mqk + T * T;                         // [T][T], s < t:  k_s . k_t
    if (!gram)  // two threads per product, whole warps per round: every lane takes part in the shuffle
      for (int id = threadIdx.x; id < 2 * T * T; id += blockDim.x) {
        int gt = 0, gsrc = id >> 1;  // T (T + 1) / 2 products k_s . q_t, then T (T - 1) / 2 products k_s . k_t
        const bool g_qk = gsrc < T * (T + 1) / 2;
        if (g_qk) {
          while (gsrc > gt) gsrc -= ++gt;
        } else {
          gsrc -= T * (T + 1) / 2;
          gt = 1;
          while (gsrc >= gt) gsrc -= gt++;
        }
        float d = 0.f;
        if (gt < cnt) {
          const float* x = (g_qk ? qs : ks) + gt * dkp;
          const float* y = ks + gsrc * dkp;
          for (int e = (id & 1) * 4; e < dkp; e += 8) {
            const float4 x4 = *reinterpret_cast<const float4*>(x + e);
            const float4 y4 = *reinterpret_cast<const float4*>(y + e);
            d = fmaf(x4.x, y4.x, d); d = fmaf(x4.y, y4.y, d); d = fmaf(x4.z, y4.z, d); d = fmaf(x4.w, y4.w, d);
          }
        }
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        if (gt < cnt && (id & 1) == 0) (g_qk ? Mqk : Mkk)[gt * T + gsrc] = d;
      }
    // A whole group is walked by code without a test per token, so that the tokens' loads and sums overlap.
    auto walk = [&](auto whole) {
      constexpr bool WHOLE = decltype(whole)::value;
      // the warp's part of the sums over the state as the group found it
#pragma unroll
      for (int t = 0; t < T; ++t)
        if (WHOLE || t < cnt) {
          const float4* kp = reinterpret_cast<const float4*>(ks + t * dkp + i0);
          const float4* qp = reinterpret_cast<const float4*>(qs + t * dkp + i0);
          float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
          for (int i = 0; i < NR; i += 4) {
            const float4 k4 = kp[i >> 2], q4 = qp[i >> 2];
            a0 = fmaf(k4.x, s[i], a0); a1 = fmaf(k4.y, s[i + 1], a1); a0 = fmaf(k4.z, s[i + 2], a0); a1 = fmaf(k4.w, s[i + 3], a1);
            b0 = fmaf(q4.x, s[i], b0); b1 = fmaf(q4.y, s[i + 1], b1); b0 = fmaf(q4.z, s[i + 2], b0); b1 = fmaf(q4.w, s[i + 3], b1);
          }
          parts[(t * W + warp) * 32 + lane] = a0 + a1;
          parts[((T + t) * W + warp) * 32 + lane] = b0 + b1;
        }
      __syncthreads();  // the parts are there
      if (WHOLE || warp < cnt) {  // this warp adds the parts of token `warp`
        float Pt = 0.f, Bt = 0.f;
#pragma unroll
        for (int w = 0; w < W; ++w) {
          Pt += parts[(warp * W + w) * 32 + lane];
          Bt += parts[((T + warp) * W + w) * 32 + lane];
        }
        sums[warp * 32 + lane] = Pt;
        sums[(T + warp) * 32 + lane] = Bt;
      }
      __syncthreads();  // P, B and the products are there
      // the writes, one after another: scalars of this column only.  ud[x] = (c_t / c_x) u_x as token t sees it.
      float ud[T];
      float c = 1.f;
#pragma unroll
      for (int t = 0; t < T; ++t) {
        ud[t] = 0.f;
        if (WHOLE || t < cnt) {
          float mk[T], mq[T];
#pragma unroll
          for (int s4 = 0; s4 < T; s4 += 4) {
            if (s4 < t) *reinterpret_cast<float4*>(mk + s4) = *reinterpret_cast<const float4*>(Mkk + t * T + s4);
            if (s4 <= t) *reinterpret_cast<float4*>(mq + s4) = *reinterpret_cast<const float4*>(Mqk + t * T + s4);
          }
          const float g = gs[t];
          c *= g;
          float a = c * sums[t * 32 + lane];
#pragma unroll
          for (int x = 0; x < t; ++x) {
            ud[x] *= g;
            a = fmaf(mk[x], ud[x], a);
          }
          ud[t] = bs[t] * (vs[t * 32 + lane] - a);
          if (t == warp) {  // this warp makes the token's o
            float ov = c * sums[(T + t) * 32 + lane];
#pragma unroll
            for (int x = 0; x <= t; ++x) ov = fmaf(mq[x], ud[x], ov);
            if (col_ok) o[((size_t)(t0 + t) * H + hd) * dv + j] = ov;
          }
        }
      }
      // the state after the group: c = the group's whole decay, ud = every write decayed by the tokens after it
#pragma unroll
      for (int i = 0; i < NR; ++i) s[i] *= c;
#pragma unroll
      for (int t = 0; t < T; ++t)
        if (WHOLE || t < cnt) {
          const float4* kp = reinterpret_cast<const float4*>(ks + t * dkp + i0);
#pragma unroll
          for (int i = 0; i < NR; i += 4) {
            const float4 k4 = kp[i >> 2];
            s[i] = fmaf(k4.x, ud[t], s[i]); s[i + 1] = fmaf(k4.y, ud[t], s[i + 1]);
            s[i + 2] = fmaf(k4.z, ud[t], s[i + 2]); s[i + 3] = fmaf(k4.w, ud[t], s[i + 3]);
          }
        }
    };
    if (cnt == T) walk(std::true_type{});
    else walk(std::false_type{});
  }
#pragma unroll
  for (int i = 0; i < NR; ++i)
    if (col_ok && i0 + i < dk) S[(size_t)(i0 + i) * dv + j] = s[i];
}

template <int NR>
static int launch_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* decay, float* state,
                             const int* cu_q, const int* slot_ids, const float* gram, float* o, int R, int G, int H, int dk, int dv,
                             cudaStream_t stream) {
  constexpr int W = DELTA_W;
  constexpr size_t smem = sizeof(float) * (2 * ((size_t)2 * DELTA_TB * W * NR + DELTA_TB * 32 + 2 * DELTA_TB + 2 * DELTA_TB * DELTA_TB) +
                                           (size_t)2 * DELTA_TB * W * 32 + 2 * DELTA_TB * 32);
  if (smem > 48 * 1024) JLX_CUDA(cudaFuncSetAttribute(delta_scan_kernel<NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  JLX_CUDA(jlx_launch_pdl(delta_scan_kernel<NR>, dim3((dv + 31) / 32, H, R), dim3(W * 32), smem, stream, q, k, v, beta, decay, state, cu_q,
                          slot_ids, gram, o, G, H, dk, dv));
  JLX_LAUNCH_CHECK("delta_scan");
  return 0;
}

// q, k: float32 [N, G, dk]; v, o: [N, H, dv]; beta, decay: [N, H]; state: float32 [slots, H, dk, dv]; gram: scratch
// float32 [N, G, 2, DELTA_TB] on a 16-byte boundary, or null (every block then makes the products of its groups itself).
JLX_API int jlx_delta_scan(const float* q, const float* k, const float* v, const float* beta, const float* decay, float* state,
                           const int* cu_q, const int* slot_ids, const int* req_of_token, float* gram, float* o, int N, int R, int G,
                           int H, int dk, int dv, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && R >= 0 && G > 0 && H > 0 && dk > 0 && dv > 0 && H % G == 0, "delta_scan: bad sizes N=%d R=%d G=%d H=%d dk=%d dv=%d", N,
              R, G, H, dk, dv);
  JLX_REQUIRE(dk <= 512, "delta_scan: key size %d is above the supported maximum 512", dk);
  JLX_REQUIRE(H <= 65535 && R <= 65535, "delta_scan: too many heads or requests");
  JLX_REQUIRE(!gram || (req_of_token && ((uintptr_t)gram & 15) == 0), "delta_scan: the products' scratch needs a 16-byte boundary and the tokens' requests");
  if (R == 0 || N == 0) return 0;
  if (N <= R) gram = nullptr;  // single tokens: one product per block, not worth a launch
  if (gram) {
    const int warps = G < 8 ? G : 8;
    JLX_CUDA(jlx_launch_pdl(delta_gram_kernel, dim3(N), dim3(warps * 32), 0, stream, q, k, cu_q, req_of_token, gram, G, dk));
    JLX_LAUNCH_CHECK("delta_gram");
  }
#define DELTA_ARGS q, k, v, beta, decay, state, cu_q, slot_ids, gram, o, R, G, H, dk, dv, stream
  const int nr = (dk + DELTA_W - 1) / DELTA_W;  // rows per warp
  if (nr <= 4) return launch_delta_scan<4>(DELTA_ARGS);
  if (nr <= 8) return launch_delta_scan<8>(DELTA_ARGS);
  if (nr <= 12) return launch_delta_scan<12>(DELTA_ARGS);
  if (nr <= 16) return launch_delta_scan<16>(DELTA_ARGS);
  if (nr <= 24) return launch_delta_scan<24>(DELTA_ARGS);
  if (nr <= 32) return launch_delta_scan<32>(DELTA_ARGS);
  if (nr <= 48) return launch_delta_scan<48>(DELTA_ARGS);
  return launch_delta_scan<64>(DELTA_ARGS);
#undef DELTA_ARGS
}
