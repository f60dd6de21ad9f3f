// Linear attention with a decay per key channel: a matrix state S [dk, dv] per request and head that every token
// decays row by row and adds an outer product to,
//
//     S_t = diag(d_t) S_(t-1) + k_t v_t^T,
//
// read either AFTER the update,  o_t = S_t^T q_t  (gated linear attention), or BEFORE it with a bonus u for the
// token itself,  o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t  (RWKV-style time mixing).  Everything here is 32-bit:
// decays, their logarithms and exponentials, the state, the sums.  The kernels:
//
//   token_shift_blend  rows m of [M, N, D]: h + (h_prev - h) * mu_m, h_prev the request's previous token (its state
//                      [D] across steps, zeros at the start); the step's last h of a request becomes its state.
//                      It can also write the row offsets m * N of the blends (groups of a grouped product).
//   decay_prep         q (scaled), k, v and the decay d of every token and head from projected rows (split-K partials
//                      are added on the way); d = exp(-exp(z + b)), sigmoid(z + b)^(1/tau), or a constant per head;
//                      optionally q and k turned by the token's position on their first entries (rotate-half pairs)
//                      before q_scale and k_scale are applied.
//   decay_scan         the recurrence over each request's tokens, in order; the state lives in registers.
//   head_norm_gate     each head's o divided by its root mean square, times a weight, times silu(gate), times a
//                      constant, written into (a column range of) the rows that the output product reads.
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

// ------------------------------------------------------------------------------------------------ token shift
// Blocks [0, R): request r's first token of the step and the move of its state (one thread per channel reads the old
// state and then writes the new one).  Blocks [R, R + N): every other token; they never touch the state.
template <typename T>
__global__ void token_shift_blend_kernel(const float* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                                         const int* __restrict__ cu_q, const int* __restrict__ slot_ids,
                                         const int* __restrict__ req_of_token, T* __restrict__ out, int N, int R, int D, int M,
                                         int* __restrict__ group_offsets) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  // the row offsets m * N of the M blends in the stacked output, for a grouped product over them
  if (group_offsets && blockIdx.x == 0 && (int)threadIdx.x <= M) group_offsets[threadIdx.x] = threadIdx.x * N;
  int n;
  const float* prev;
  float* st = nullptr;
  int last = 0;
  if ((int)blockIdx.x < R) {
    const int r = blockIdx.x;
    n = cu_q[r];
    last = cu_q[r + 1] - 1;
    if (last < n) return;
    st = state + (size_t)slot_ids[r] * D;
    prev = st;
  } else {
    n = blockIdx.x - R;
    if (n == cu_q[req_of_token[n]]) return;  // a first token: served by its request's block
    prev = h + (size_t)(n - 1) * D;
  }
  const float* cur = h + (size_t)n * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float c = cur[d], p = prev[d];
    const float diff = p - c;
    for (int m = 0; m < M; ++m) out[((size_t)m * N + n) * D + d] = from_f32<T>(fmaf(diff, mu[(size_t)m * D + d], c));
    if (st) st[d] = h[(size_t)last * D + d];
  }
}

JLX_API int jlx_token_shift_blend(const float* h, const float* mu, float* state, const int* cu_q, const int* slot_ids,
                                  const int* req_of_token, void* out, int out_dtype, int N, int R, int D, int M,
                                  int* group_offsets, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && R >= 0 && D > 0 && M >= 1 && M < 64, "token_shift_blend: bad sizes N=%d R=%d D=%d M=%d", N, R, D, M);
  if (N == 0) return 0;
  const int threads = D >= 1024 ? 256 : 128;
  JLX_DISPATCH_DTYPE(out_dtype, T, {
    JLX_CUDA(jlx_launch_pdl(token_shift_blend_kernel<T>, dim3(R + N), dim3(threads), 0, stream, h, mu, state, cu_q, slot_ids,
                            req_of_token, (T*)out, N, R, D, M, group_offsets));
  });
  JLX_LAUNCH_CHECK("token_shift_blend");
  return 0;
}

// ------------------------------------------------------------------------------------------------ decay prep
// DECAY_HEAD_CONSTANT: one fixed decay per head (head_decay [H]) for all its key channels and every token; z unused.
enum { DECAY_DOUBLE_EXP = 0, DECAY_SIGMOID_POWER = 1, DECAY_HEAD_CONSTANT = 2 };

// One block per (token, head).
__global__ void decay_prep_kernel(RowsView q, RowsView k, RowsView v, RowsView z, const float* __restrict__ z_bias, int mode,
                                  float inv_tau, float q_scale, float* __restrict__ qo, float* __restrict__ ko,
                                  float* __restrict__ d_out, float* __restrict__ vo, int H, int dk, int dv,
                                  const float* __restrict__ head_decay, float k_scale, const float* __restrict__ inv_freq, int rot,
                                  const int* __restrict__ positions) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t n = blockIdx.x;
  const int hd = blockIdx.y;
  const size_t at_k = (n * H + hd) * dk, at_v = (n * H + hd) * dv;
  const int half = rot >> 1;
  const float pos = rot > 0 ? (float)positions[n] : 0.f;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) {
    const int c = hd * dk + i;
    float qv = rows_at(q, n, c), kv = rows_at(k, n, c);
    if (i < rot) {  // entry i turns with entry i +- rot / 2 by the angle position * inv_freq[i mod rot / 2]
      const bool first = i < half;
      const int partner = first ? c + half : c - half;
      float sn, cs;
      sincosf(pos * inv_freq[first ? i : i - half], &sn, &cs);
      const float qp = rows_at(q, n, partner), kp = rows_at(k, n, partner);
      qv = first ? qv * cs - qp * sn : qv * cs + qp * sn;
      kv = first ? kv * cs - kp * sn : kv * cs + kp * sn;
    }
    qo[at_k + i] = qv * q_scale;
    ko[at_k + i] = kv * k_scale;
    if (mode == DECAY_HEAD_CONSTANT) {
      d_out[at_k + i] = head_decay[hd];
      continue;
    }
    const float x = rows_at(z, n, c) + (z_bias ? z_bias[c] : 0.f);
    float d;
    if (mode == DECAY_DOUBLE_EXP) {
      d = expf(-expf(x));
    } else {
      // sigmoid(x)^(1/tau) = exp(-softplus(-x) / tau), softplus(y) = max(y, 0) + log1p(exp(-|y|))
      const float sp = fmaxf(-x, 0.f) + log1pf(expf(-fabsf(x)));
      d = expf(-sp * inv_tau);
    }
    d_out[at_k + i] = d;
  }
  for (int j = threadIdx.x; j < dv; j += blockDim.x) vo[at_v + j] = rows_at(v, n, hd * dv + j);
}

JLX_API int jlx_decay_prep(const RowsView* q, const RowsView* k, const RowsView* v, const RowsView* z, const float* z_bias,
                           int mode, float tau, float q_scale, float* qo, float* ko, float* d_out, float* vo, int N, int H,
                           int dk, int dv, const float* head_decay, float k_scale, const float* inv_freq, int rot,
                           const int* positions, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && dk > 0 && dv > 0 && H <= 65535, "decay_prep: bad sizes N=%d H=%d dk=%d dv=%d", N, H, dk, dv);
  JLX_REQUIRE(mode == DECAY_DOUBLE_EXP || (mode == DECAY_SIGMOID_POWER && tau > 0.f) || (mode == DECAY_HEAD_CONSTANT && head_decay),
              "decay_prep: unknown decay form, tau <= 0, or the heads' constant decays are missing");
  JLX_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dk && (rot == 0 || (inv_freq && positions)), "decay_prep: %d rotated entries of %d need frequencies and positions", rot, dk);
  RowsView none = {nullptr, 0, 0, 0, 0};
  if (!z) z = &none;
  if (N == 0) return 0;
  JLX_CUDA(jlx_launch_pdl(decay_prep_kernel, dim3(N, H), dim3(dk + dv >= 256 ? 128 : 64), 0, stream, *q, *k, *v, *z, z_bias, mode,
                          mode == DECAY_SIGMOID_POWER ? 1.f / tau : 0.f, q_scale, qo, ko, d_out, vo, H, dk, dv, head_decay, k_scale, inv_freq, rot, positions));
  JLX_LAUNCH_CHECK("decay_prep");
  return 0;
}

// ------------------------------------------------------------------------------------------------ the recurrence
// One block per (request, head, slice of 32 value columns).  Lane = a value column; warp w keeps rows [w NR, (w+1) NR)
// of S for that column in registers.  The tokens' q, k, d rows and v slice come through shared memory SCAN_TB tokens
// at a time, two buffers taking turns: while a group of tokens is walked, asynchronous copies bring the next.  Between
// two barriers a warp walks a group (o does not feed back into S), reading its rows' q, k, d four at a time, and leaves
// its part of each o; the parts are added in warp order.  A token's sums run in the same order wherever it stands in a
// step, so portions give bit for bit what whole prompts give.
#define SCAN_TB 16

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// G: row groups within a warp.  With G = 1 a lane is one of 32 value columns and holds NR rows; with G = 2 or 4 a block
// serves 16 or 8 columns, and a warp's lanes split its NR rows between them (NR / G each), their parts of o meeting in
// shuffles.  More, lighter blocks: a model with few heads still fills the GPU with one request.  G is chosen from the
// model's sizes alone (never from the batch), so a token's sums do not change with what else is in the step.
template <int NR, int G, bool READ_AFTER>
__global__ void decay_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ d,
                                  const float* __restrict__ v, const float* __restrict__ u, float* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ slot_ids, float* __restrict__ o,
                                  int H, int dk, int dv) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  constexpr int CW = 32 / G, RL = NR / G;
  static_assert(RL >= 4 && RL % 4 == 0, "a lane reads its rows four at a time");
  extern __shared__ __align__(16) float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const int cl = lane % CW, rg = lane / CW;
  const int dkp = W * NR;
  const int stage_floats = 3 * SCAN_TB * dkp + SCAN_TB * 32;  // [q | k | d][SCAN_TB][dkp], v [SCAN_TB][32] (CW in use)
  float* part = smem + 2 * stage_floats;                     // [SCAN_TB][W][CW]
  const int r = blockIdx.x, hd = blockIdx.y, j0 = blockIdx.z * CW;
  const int j = j0 + cl;
  const bool col = j < dv;
  const int i0 = warp * NR + rg * RL;
  float uu[RL];
#pragma unroll
  for (int ii = 0; ii < RL; ++ii) uu[ii] = (!READ_AFTER && u && i0 + ii < dk) ? u[hd * dk + i0 + ii] : 0.f;
  // what no copy ever writes: rows beyond dk (q = k = 0, d = 1) and value columns beyond dv (0)
  for (int b = 0; b < 2; ++b) {
    float* st = smem + b * stage_floats;
    for (int idx = threadIdx.x; idx < SCAN_TB * dkp; idx += blockDim.x)
      if (idx % dkp >= dk) {
        st[idx] = 0.f;
        st[SCAN_TB * dkp + idx] = 0.f;
        st[2 * SCAN_TB * dkp + idx] = 1.f;
      }
    for (int idx = threadIdx.x; idx < SCAN_TB * 32; idx += blockDim.x)
      if (j0 + (idx & 31) >= dv) st[3 * SCAN_TB * dkp + idx] = 0.f;
  }
  pdl_wait();
  const int n0 = cu_q[r], n1 = cu_q[r + 1];
  if (n1 <= n0) return;
  float* S = state + ((size_t)slot_ids[r] * H + hd) * dk * dv;
  float s[RL];
#pragma unroll
  for (int ii = 0; ii < RL; ++ii) s[ii] = (col && i0 + ii < dk) ? S[(size_t)(i0 + ii) * dv + j] : 0.f;

  // 16-byte copies where every row starts on a 16-byte boundary
  const bool vec = (dk & 3) == 0 && (dv & 3) == 0 && ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)d | (uintptr_t)v) & 15) == 0);
  const int nv = min(CW, dv - j0);
  auto stage = [&](int t0, int b) {  // asynchronous copies of the group's rows into buffer b
    float* st = smem + b * stage_floats;
    const int cnt = min(SCAN_TB, n1 - t0);
    if (vec) {
      const int dk4 = dk >> 2, nv4 = nv >> 2;
      for (int idx = threadIdx.x; idx < cnt * dk4; idx += blockDim.x) {
        const int tt = idx / dk4, i = (idx - tt * dk4) << 2;
        const size_t at = ((size_t)(t0 + tt) * H + hd) * dk + i;
        float* dst = st + tt * dkp + i;
        cp_async16(dst, q + at);
        cp_async16(dst + SCAN_TB * dkp, k + at);
        cp_async16(dst + 2 * SCAN_TB * dkp, d + at);
      }
      for (int idx = threadIdx.x; idx < cnt * nv4; idx += blockDim.x) {
        const int tt = idx / nv4, l = (idx - tt * nv4) << 2;
        cp_async16(st + 3 * SCAN_TB * dkp + tt * 32 + l, v + ((size_t)(t0 + tt) * H + hd) * dv + j0 + l);
      }
      cp_async_commit();
      return;
    }
    for (int idx = threadIdx.x; idx < cnt * dk; idx += blockDim.x) {
      const int tt = idx / dk, i = idx - tt * dk;
      const size_t at = ((size_t)(t0 + tt) * H + hd) * dk + i;
      float* dst = st + tt * dkp + i;
      cp_async4(dst, q + at);
      cp_async4(dst + SCAN_TB * dkp, k + at);
      cp_async4(dst + 2 * SCAN_TB * dkp, d + at);
    }
    for (int idx = threadIdx.x; idx < cnt * nv; idx += blockDim.x) {
      const int tt = idx / nv, l = idx - tt * nv;
      cp_async4(st + 3 * SCAN_TB * dkp + tt * 32 + l, v + ((size_t)(t0 + tt) * H + hd) * dv + j0 + l);
    }
    cp_async_commit();
  };

  stage(n0, 0);
  int b = 0;
  for (int t0 = n0; t0 < n1; t0 += SCAN_TB, b ^= 1) {
    const int cnt = min(SCAN_TB, n1 - t0);
    const bool more = t0 + SCAN_TB < n1;
    if (more) {
      stage(t0 + SCAN_TB, b ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();  // this group's rows are there; the parts of the group before are consumed
    const float* st = smem + b * stage_floats;
    // unrolled, so that the next tokens' reads from shared memory are in flight while a token's sums are made
#pragma unroll 4
    for (int tt = 0; tt < cnt; ++tt) {
      const float vj = st[3 * SCAN_TB * dkp + tt * 32 + cl];
      const float4* qt = reinterpret_cast<const float4*>(st + tt * dkp + i0);
      const float4* kt = reinterpret_cast<const float4*>(st + SCAN_TB * dkp + tt * dkp + i0);
      const float4* dt = reinterpret_cast<const float4*>(st + 2 * SCAN_TB * dkp + tt * dkp + i0);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i4 = 0; i4 < RL / 4; ++i4) {
        const float4 q4 = qt[i4], k4 = kt[i4], d4 = dt[i4];
        const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int ii = 4 * i4 + c;
          const float kv = kk[c] * vj;
          if (READ_AFTER) {
            s[ii] = fmaf(dd[c], s[ii], kv);
            acc[c] = fmaf(qq[c], s[ii], acc[c]);
          } else {
            acc[c] = fmaf(qq[c], fmaf(uu[ii], kv, s[ii]), acc[c]);
            s[ii] = fmaf(dd[c], s[ii], kv);
          }
        }
      }
      float total = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      if (G == 4) total += __shfl_xor_sync(0xffffffffu, total, 8);
      if (G >= 2) total += __shfl_xor_sync(0xffffffffu, total, 16);
      if (rg == 0) part[(tt * W + warp) * CW + cl] = total;
    }
    __syncthreads();  // the parts are there; this group's rows are consumed
    for (int idx = threadIdx.x; idx < cnt * CW; idx += blockDim.x) {
      const int tt = idx / CW, l = idx % CW;
      float sum = 0.f;
      for (int w = 0; w < W; ++w) sum += part[(tt * W + w) * CW + l];
      if (j0 + l < dv) o[((size_t)(t0 + tt) * H + hd) * dv + j0 + l] = sum;
    }
  }
#pragma unroll
  for (int ii = 0; ii < RL; ++ii)
    if (col && i0 + ii < dk) S[(size_t)(i0 + ii) * dv + j] = s[ii];
}

template <int NR, int G, bool READ_AFTER>
static int launch_decay_scan(const float* q, const float* k, const float* d, const float* v, const float* u, float* state,
                             const int* cu_q, const int* slot_ids, float* o, int R, int H, int dk, int dv, cudaStream_t stream) {
  const int W = (dk + NR - 1) / NR, CW = 32 / G;
  const size_t smem = sizeof(float) * (2 * ((size_t)3 * SCAN_TB * W * NR + SCAN_TB * 32) + (size_t)SCAN_TB * W * CW);
  if (smem > 48 * 1024)
    JLX_CUDA(cudaFuncSetAttribute(decay_scan_kernel<NR, G, READ_AFTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  JLX_CUDA(jlx_launch_pdl(decay_scan_kernel<NR, G, READ_AFTER>, dim3(R, H, (dv + CW - 1) / CW), dim3(W * 32), smem, stream, q, k, d, v,
                          u, state, cu_q, slot_ids, o, H, dk, dv));
  JLX_LAUNCH_CHECK("decay_scan");
  return 0;
}

// Blocks that one request gives with G row groups per warp; enough of them (SCAN_FILL) fill the GPU.
#define SCAN_FILL 128
static int scan_row_groups(int H, int dv, int nr) {
  if (H * ((dv + 31) / 32) >= SCAN_FILL || nr < 8) return 1;
  if (H * ((dv + 15) / 16) >= SCAN_FILL || nr < 16) return 2;
  return 4;
}

// q, k, d: float32 [N, H, dk]; v: [N, H, dv]; u: [H, dk] or null (only read before the update); state: [slots, H, dk, dv];
// o: [N, H, dv].  read_after: 1 = o_t = S_t^T q_t;  0 = o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t.
JLX_API int jlx_decay_scan(const float* q, const float* k, const float* d, const float* v, const float* u, float* state,
                           const int* cu_q, const int* slot_ids, float* o, int R, int H, int dk, int dv, int read_after,
                           cudaStream_t stream) {
  JLX_REQUIRE(R >= 0 && H > 0 && dk > 0 && dv > 0, "decay_scan: bad sizes R=%d H=%d dk=%d dv=%d", R, H, dk, dv);
  JLX_REQUIRE(dk <= 512, "decay_scan: %d key channels per head; up to 512 are supported", dk);
  JLX_REQUIRE(H <= 65535 && (dv + 7) / 8 <= 65535, "decay_scan: too many heads or value columns");
  if (R == 0) return 0;
#define JLX_SCAN_ARGS q, k, d, v, u, state, cu_q, slot_ids, o, R, H, dk, dv, stream
#define JLX_SCAN(NR, G) return read_after ? launch_decay_scan<NR, G, true>(JLX_SCAN_ARGS) : launch_decay_scan<NR, G, false>(JLX_SCAN_ARGS)
#define JLX_SCAN_G(NR)                        \
  {                                           \
    const int g = scan_row_groups(H, dv, NR); \
    if (g == 4) { JLX_SCAN(NR, 4); }          \
    if (g == 2) { JLX_SCAN(NR, 2); }          \
    JLX_SCAN(NR, 1);                          \
  }
  if (dk <= 32) {
    if (scan_row_groups(H, dv, 8) >= 2) { JLX_SCAN(8, 2); }
    JLX_SCAN(8, 1);
  }
  if (dk <= 128) JLX_SCAN_G(16)
  if (dk <= 256) JLX_SCAN_G(32)
  JLX_SCAN_G(64)
#undef JLX_SCAN_G
#undef JLX_SCAN
#undef JLX_SCAN_ARGS
}

// ------------------------------------------------------------------------------------------------ head norm + gate
// One block per (token, head): out[n, h dv + c] = mult * o[c] / sqrt(mean(o^2) + eps) * weight[(per_head ? h dv : 0) + c]
// * silu(gate[n, h dv + c]).  weight and gate may be null.  out's rows are ld_out elements apart.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, int per_head, RowsView gate,
                                      float eps, float mult, T* __restrict__ out, long long ld_out, int H, int dv) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t n = blockIdx.x;
  const int hd = blockIdx.y;
  const float* row = o + (n * H + hd) * dv;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)dv + eps);
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float y = row[c] / rms;
    if (weight) y *= weight[(per_head ? hd * dv : 0) + c];
    if (gate.p) {
      const float g = rows_at(gate, n, hd * dv + c);
      y *= g / (1.f + expf(-g));
    }
    out[n * ld_out + hd * dv + c] = from_f32<T>(mult * y);
  }
}

JLX_API int jlx_head_norm_gate(const float* o, const float* weight, int per_head, const RowsView* gate, float eps, float mult,
                               void* out, int out_dtype, long long ld_out, int N, int H, int dv, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && H > 0 && dv > 0 && H <= 65535 && ld_out >= (long long)H * dv, "head_norm_gate: bad sizes");
  JLX_REQUIRE(eps > 0.f, "head_norm_gate: eps must be positive");
  if (N == 0) return 0;
  RowsView none = {nullptr, 0, 0, 1, 0};
  const int threads = dv > 128 ? 128 : (dv > 32 ? 64 : 32);
  JLX_DISPATCH_DTYPE(out_dtype, T, {
    JLX_CUDA(jlx_launch_pdl(head_norm_gate_kernel<T>, dim3(N, H), dim3(threads), 0, stream, o, weight, per_head,
                            gate ? *gate : none, eps, mult, (T*)out, ld_out, H, dv));
  });
  JLX_LAUNCH_CHECK("head_norm_gate");
  return 0;
}
