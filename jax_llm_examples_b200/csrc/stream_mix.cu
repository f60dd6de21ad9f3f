// Several residual streams per token ("hyper-connections"): instead of one row x a token carries S rows x_1 .. x_S.
// A sublayer reads a weighted sum of them, and its output y goes back into every stream while the streams mix:
//
//     x_t <- sum_s mix[s, t] x_s + out[t] y        (all t at once, from the old rows; mix is indexed [from, to])
//     u    = sum_t in[t] x_t                       (what the NEXT sublayer reads)
//     h    = gamma * u / sqrt(mean(u^2) + eps)     (its norm)
//
// stream_mix_norm does all three in one pass over a token's rows: the write-back of the sublayer that just ran (y may
// still be split-K partials, added in ascending order), the read of the next one and its RMS norm.  It is what the
// residual-add + norm kernel is to a single stream.  Without a pending y it only reads and norms; with `in` null the
// read is the plain sum of the streams (what the model's final norm sees).  Everything is 32-bit; only `out` may be
// rounded.  One block per token; every sum runs in an order fixed by the channel alone, so a token's result does not
// depend on the batch.
#include "common.cuh"

#define STREAMS_MAX 16

struct StreamMixArgs {
  float* x;               // [N, S, D] streams, updated in place (not written when rows are gathered)
  const float* x_first;   // optional [N, D]: the streams have not been written yet and all equal this row
  const float* y;         // optional pending sublayer output, [splits][N][D]
  long long y_stride;
  int y_splits;
  const float* mix;       // [S, S] of the pending sublayer (with y)
  const float* out_w;     // [S]
  const float* in_w;      // [S] of the next sublayer, or null: ones
  const float* gamma;     // [D] or null
  float eps;
  const int* row_index;   // optional: row n reads source row row_index[n]; x is not written back
  float* sum_out;         // optional [N, D]: the plain sum of the (new) streams
  int S, D;
};

// V consecutive channels of a row as one access (V = 4 needs D % 4 == 0 and 16-byte aligned rows).
template <int V> struct Chan { float v[V]; };
template <int V> __device__ __forceinline__ Chan<V> load_chan(const float* p) {
  Chan<V> c;
  if (V == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    c.v[0] = t.x; c.v[1 % V] = t.y; c.v[2 % V] = t.z; c.v[3 % V] = t.w;
  } else {
    c.v[0] = *p;
  }
  return c;
}
template <int V> __device__ __forceinline__ void store_chan(float* p, const Chan<V>& c) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(c.v[0], c.v[1 % V], c.v[2 % V], c.v[3 % V]);
  else *p = c.v[0];
}

// MAXS: the stream count rounded up to 2, 4, 8 or 16 (a token's rows of V channels live in registers).  A channel's
// sums run in the same order for V = 1 and V = 4.
template <typename T, int MAXS, int V>
__global__ void __launch_bounds__(512) stream_mix_norm_kernel(StreamMixArgs a, T* __restrict__ out, float* __restrict__ out32) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  extern __shared__ __align__(16) float u_row[];  // [D]
  __shared__ float scratch[33];
  __shared__ float w_mix[MAXS * MAXS], w_out[MAXS], w_in[MAXS];
  const int S = a.S, D = a.D;
  // the small weights are the model's: read before the wait
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) w_mix[i] = a.y ? a.mix[i] : 0.f;
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    w_out[i] = a.y ? a.out_w[i] : 0.f;
    w_in[i] = a.in_w ? a.in_w[i] : 1.f;
  }
  __syncthreads();
  pdl_wait();
  const size_t n = blockIdx.x;
  const size_t r = a.row_index ? (size_t)a.row_index[n] : n;
  float* xr = a.x + r * (size_t)S * D;
  float ss = 0.f;
  for (int d = threadIdx.x * V; d < D; d += blockDim.x * V) {
    Chan<V> xs[MAXS];
    if (a.x_first) {
      const Chan<V> c = load_chan<V>(a.x_first + r * D + d);
#pragma unroll
      for (int s = 0; s < MAXS; ++s) xs[s] = c;
    } else {
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) xs[s] = load_chan<V>(xr + (size_t)s * D + d);
    }
    Chan<V> u, total, y;
#pragma unroll
    for (int i = 0; i < V; ++i) u.v[i] = total.v[i] = y.v[i] = 0.f;
    if (a.y) {
      for (int z = 0; z < a.y_splits; ++z) {
        const Chan<V> c = load_chan<V>(a.y + (size_t)z * a.y_stride + r * D + d);
#pragma unroll
        for (int i = 0; i < V; ++i) y.v[i] += c.v[i];
      }
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t < S) {
          Chan<V> v;
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
              if (s < S) acc = fmaf(w_mix[s * S + t], xs[s].v[i], acc);
            acc = fmaf(w_out[t], y.v[i], acc);
            v.v[i] = acc;
            u.v[i] = fmaf(w_in[t], acc, u.v[i]);
            total.v[i] += acc;
          }
          if (!a.row_index) store_chan<V>(xr + (size_t)t * D + d, v);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t < S) {
          if (a.x_first && !a.row_index) store_chan<V>(xr + (size_t)t * D + d, xs[t]);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            u.v[i] = fmaf(w_in[t], xs[t].v[i], u.v[i]);
            total.v[i] += xs[t].v[i];
          }
        }
      }
    }
    if (a.sum_out) store_chan<V>(a.sum_out + n * D + d, total);
    store_chan<V>(u_row + d, u);
#pragma unroll
    for (int i = 0; i < V; ++i) ss = fmaf(u.v[i], u.v[i], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)D + a.eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float v = u_row[d] * inv * (a.gamma ? a.gamma[d] : 1.f);
    if (out) out[n * D + d] = from_f32<T>(v);
    if (out32) out32[n * D + d] = v;
  }
}

// x: float32 [N, S, D]; x_first: optional float32 [N, D] (the streams' common first value; x is then written, not read);
// y: optional float32 partials of the pending sublayer output with mix [S, S] and out_w [S]; in_w: [S] or null (ones);
// gamma: [D] or null; out (out_dtype) and/or out32: [n, D]; row_index: optional int32 [n]; sum_out: optional [n, D].
JLX_API int jlx_stream_mix_norm(float* x, const float* x_first, const float* y, int y_splits, long long y_stride, const float* mix,
                                const float* out_w, const float* in_w, const float* gamma, float eps, void* out, int out_dtype,
                                float* out32, const int* row_index, float* sum_out, int n, int S, int D, cudaStream_t stream) {
  JLX_REQUIRE(n >= 0 && D > 0 && S >= 1 && S <= STREAMS_MAX, "stream_mix_norm: %d streams of width %d; 1..%d streams are supported", S, D, STREAMS_MAX);
  JLX_REQUIRE(!y || (mix && out_w && y_splits >= 1), "stream_mix_norm: a pending output needs its mix matrix and its write weights");
  JLX_REQUIRE(!(y && x_first), "stream_mix_norm: streams that were never written have no pending output");
  const size_t smem = sizeof(float) * (size_t)D;
  JLX_REQUIRE(smem <= 200 * 1024, "stream_mix_norm: a row of %d does not fit shared memory", D);
  if (n == 0) return 0;
  StreamMixArgs a;
  a.x = x; a.x_first = x_first; a.y = y; a.y_stride = y_stride; a.y_splits = y_splits; a.mix = mix; a.out_w = out_w; a.in_w = in_w;
  a.gamma = gamma; a.eps = eps; a.row_index = row_index; a.sum_out = sum_out; a.S = S; a.D = D;
  const int threads = D >= 4096 ? 512 : (D >= 1024 ? 256 : 128);
  // four channels per access where every row starts on a 16-byte boundary
  const bool wide = D % 4 == 0 && y_stride % 4 == 0 &&
                    (((uintptr_t)x | (uintptr_t)x_first | (uintptr_t)y | (uintptr_t)sum_out) & 15) == 0;
#define JLX_STREAMS_V(MAXS, V)                                                                                                       \
  JLX_DISPATCH_DTYPE(out_dtype, T, {                                                                                                \
    if (smem > 48 * 1024)                                                                                                           \
      JLX_CUDA(cudaFuncSetAttribute(stream_mix_norm_kernel<T, MAXS, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
    JLX_CUDA(jlx_launch_pdl(stream_mix_norm_kernel<T, MAXS, V>, dim3(n), dim3(threads), smem, stream, a, (T*)out, out32));          \
  })
#define JLX_STREAMS(MAXS) do { if (wide) { JLX_STREAMS_V(MAXS, 4); } else { JLX_STREAMS_V(MAXS, 1); } } while (0)
  if (S <= 2) JLX_STREAMS(2);
  else if (S <= 4) JLX_STREAMS(4);
  else if (S <= 8) JLX_STREAMS(8);
  else JLX_STREAMS_V(16, 1);
#undef JLX_STREAMS
#undef JLX_STREAMS_V
  JLX_LAUNCH_CHECK("stream_mix_norm");
  return 0;
}
