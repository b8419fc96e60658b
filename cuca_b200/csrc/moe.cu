// A routed feed-forward: every token goes to the `top` experts with the largest router logits.
//   moe_route        per token: the chosen experts (largest logit first, the lower number on a tie), their weights
//                    (a softmax of just those logits) and, optionally, the weights spread over all experts
//   moe_act_dense    a[t, e, f] = relu(u[t, e, f])^2 * weight[t, e]: all experts' up-projections at once, the ones a
//                    token did not choose weighted 0, so that one contraction over (e, f) is the weighted sum
//   moe_up_sparse / moe_down_sparse   few tokens: only the chosen experts' weights are read, a warp per output
//   moe_route_scored scores are a softmax over ALL router outputs; the choice goes by score + a correction per output,
//                    the weights are the chosen scores over their sum; the last outputs may stand for experts that
//                    return their input (their weights are summed per token for `moe_identity_add`)
//   moe_glu_dense    a[t, c] = silu(g[t, c]) u[t, c] * weight[t, expert of c]: gated experts, and behind them the
//                    columns of a shared expert that every token uses with weight 1
// Routing arithmetic is 32-bit. A token's experts are summed in a fixed order, whatever else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int MAX_TOP = 32;
constexpr int MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int T, int E, int top, int* __restrict__ idx,
                 float* __restrict__ wts, float* __restrict__ dense) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* z = logits + (size_t)t * E;
  unsigned taken = 0;  // bit j: this lane's expert lane + 32 j is chosen already
  float my_z = 0.f;    // lane j keeps the j-th chosen logit
  int my_e = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int be = 0x7fffffff;
    for (int k = 0; lane + 32 * k < E; ++k) {
      const int e = lane + 32 * k;
      float v = z[e];
      v = v == v ? v : -INFINITY;  // a row of padding may hold anything: every lane must still see one order
      if (!((taken >> k) & 1u) && (v > best || (v == best && e < be) || be == 0x7fffffff)) { best = v; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > best || (ov == best && oe < be))) { best = ov; be = oe; }
    }
    if (be < E && (be & 31) == lane) taken |= 1u << (be >> 5);
    if (lane == j) { my_z = best; my_e = be < E ? be : 0; }
  }
  const float zmax = __shfl_sync(0xffffffffu, my_z, 0);
  const float p = lane < top ? expf(my_z - zmax) : 0.f;
  const float w = p / warp_sum(p);
  if (dense)
    for (int e = lane; e < E; e += 32) dense[(size_t)t * E + e] = 0.f;
  __syncwarp();
  if (lane < top) {
    idx[(size_t)t * top + lane] = my_e;
    wts[(size_t)t * top + lane] = w;
    if (dense) dense[(size_t)t * E + my_e] = w;
  }
}

template <typename T>
__global__ void moe_act_dense_kernel(const T* __restrict__ u, const float* __restrict__ dense, T* __restrict__ a,
                                     size_t n, int E, int F) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / ((size_t)E * F);
    const int e = (int)((i / F) % E);
    const float w = dense[t * E + e];
    const float v = fmaxf(to_f32(u[i]), 0.f);
    a[i] = from_f32<T>(w == 0.f ? 0.f : v * v * w);
  }
}

// Scores over all E router outputs; `top` chosen by score + correction (the lower number on a tie); weights
// s / (sum of the chosen s + 1e-20). Outputs from n_real on are identity experts: their chosen weights are summed in
// ident[t]. A warp per token; lane l holds outputs l, l + 32, ...
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int T, int E, int n_real,
                        int top, int* __restrict__ idx, float* __restrict__ wts, float* __restrict__ dense,
                        float* __restrict__ ident) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* z = logits + (size_t)t * E;
  float zmax = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    const float v = z[e];
    zmax = fmaxf(zmax, v == v ? v : -INFINITY);
  }
  zmax = warp_max(zmax);
  if (zmax == -INFINITY) zmax = 0.f;  // a row of padding may hold anything
  float total = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = z[e];
    total += v == v ? expf(v - zmax) : 0.f;
  }
  total = warp_sum(total);
  const float inv_total = total > 0.f ? 1.f / total : 0.f;
  unsigned taken = 0;
  float my_s = 0.f;
  int my_e = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY, best_s = 0.f;
    int be = 0x7fffffff;
    for (int k = 0; lane + 32 * k < E; ++k) {
      const int e = lane + 32 * k;
      const float v = z[e];
      const float sc = v == v ? expf(v - zmax) * inv_total : 0.f;
      float c = sc + (correction ? correction[e] : 0.f);
      c = c == c ? c : -INFINITY;
      if (!((taken >> k) & 1u) && (c > best || (c == best && e < be) || be == 0x7fffffff)) { best = c; be = e; best_s = sc; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > best || (ov == best && oe < be))) { best = ov; be = oe; best_s = os; }
    }
    if (be < E && (be & 31) == lane) taken |= 1u << (be >> 5);
    if (lane == j) { my_s = best_s; my_e = be < E ? be : 0; }
  }
  const float chosen = warp_sum(lane < top ? my_s : 0.f);
  const float w = my_s / (chosen + 1e-20f);
  const float iw = warp_sum(lane < top && my_e >= n_real ? w : 0.f);
  if (dense)
    for (int e = lane; e < E; e += 32) dense[(size_t)t * E + e] = 0.f;
  __syncwarp();
  if (lane < top) {
    idx[(size_t)t * top + lane] = my_e;
    wts[(size_t)t * top + lane] = w;
    if (dense) dense[(size_t)t * E + my_e] = w;
  }
  if (ident && lane == 0) ident[t] = iw;
}

// gu: [T, 2 C] (gates, then ups); a[t, c] = silu(g) u w with w = dense[t, c / F] for c < EF (ld_dense outputs a row),
// 1 for the columns behind (a shared expert).
template <typename T>
__global__ void moe_glu_dense_kernel(const T* __restrict__ gu, const float* __restrict__ dense, int ld_dense,
                                     T* __restrict__ a, size_t n, int C, int EF, int F) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / C;
    const int c = (int)(i % C);
    const float w = c < EF ? dense[t * ld_dense + c / F] : 1.f;
    const float g = to_f32(gu[t * 2 * C + c]), u = to_f32(gu[t * 2 * C + C + c]);
    a[i] = from_f32<T>(w == 0.f ? 0.f : g / (1.f + expf(-g)) * u * w);
  }
}

// The same, 16 bytes a thread (V values of one expert: F, EF and C are multiples of V).
template <typename T, int V>
__global__ void moe_glu_dense_vec_kernel(const T* __restrict__ gu, const float* __restrict__ dense, int ld_dense,
                                         T* __restrict__ a, size_t n_vec, int C, int EF, int F) {
  pdl_trigger();
  pdl_wait();
  const int cv = C / V;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / cv;
    const int c = (int)(i % cv) * V;
    const float w = c < EF ? dense[t * ld_dense + c / F] : 1.f;
    uint4 out4 = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {  // (an expert the token did not choose: its rows are not read)
      const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * C + c);
      const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * C + C + c);
      const T* g = reinterpret_cast<const T*>(&g4);
      const T* u = reinterpret_cast<const T*>(&u4);
      T* o = reinterpret_cast<T*>(&out4);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float gv = to_f32(g[e]);
        o[e] = from_f32<T>(gv / (1.f + expf(-gv)) * to_f32(u[e]) * w);
      }
    }
    *reinterpret_cast<uint4*>(a + t * C + c) = out4;
  }
}

// y[t] (+)= ident[t] * h[t]: the experts that return their input.
template <typename T>
__global__ void moe_identity_add_kernel(float* __restrict__ y, const T* __restrict__ h, const float* __restrict__ ident,
                                        int store, size_t n, int N) {
  pdl_trigger();
  pdl_wait();
  if ((N & 3) == 0 && ((uintptr_t)y & 15) == 0) {  // four values a thread
    const size_t n4 = n / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
      const float w = ident[(i * 4) / N];
      float4 v = store ? make_float4(0.f, 0.f, 0.f, 0.f) : reinterpret_cast<const float4*>(y)[i];
      const T* hv = h + i * 4;
      v.x += w * to_f32(hv[0]); v.y += w * to_f32(hv[1]); v.z += w * to_f32(hv[2]); v.w += w * to_f32(hv[3]);
      reinterpret_cast<float4*>(y)[i] = v;
    }
    return;
  }
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = ident[i / N] * to_f32(h[i]);
    y[i] = store ? v : y[i] + v;
  }
}

// A warp's dot product of two rows of n values: 16 bytes a lane at a time where the rows allow it.
__device__ __forceinline__ float warp_dot(const float* w, const float* x, int n, int lane) {
  float acc = 0.f;
  for (int i = lane; i < n; i += 32) acc = fmaf(w[i], x[i], acc);
  return warp_sum(acc);
}
__device__ __forceinline__ float warp_dot(const __nv_bfloat16* w, const __nv_bfloat16* x, int n, int lane) {
  float acc = 0.f;
  if (n % 8 == 0 && ((((uintptr_t)w) | ((uintptr_t)x)) & 15) == 0) {
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(w + i), b = *reinterpret_cast<const uint4*>(x + i);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 fa = __bfloat1622float2(pa[k]), fb = __bfloat1622float2(pb[k]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) acc = fmaf(__bfloat162float(w[i]), __bfloat162float(x[i]), acc);
  }
  return warp_sum(acc);
}

// a[pair, f] = act(W[e(pair)] . h[t]) * weight(pair); pair = t * top + j. GLU false: W_up [E F, K], act = relu(.)^2.
// GLU true: w_up holds every expert's gate rows and, `up_rows` rows further on, its up rows; act = silu(gate) up.
// A pair whose expert number is n_real or more has no weights (it returns its input): nothing is written for it.
template <typename T, bool GLU>
__global__ void __launch_bounds__(256)
moe_up_sparse_kernel(const T* __restrict__ h, const T* __restrict__ w_up, const int* __restrict__ idx,
                     const float* __restrict__ wts, T* __restrict__ a, int top, int F, int K, int n_real, size_t up_rows) {
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.y, f = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (f >= F) return;
  const int e = idx[pair];
  if (e >= n_real) return;
  const T* wr = w_up + ((size_t)e * F + f) * K;
  const T* hr = h + (size_t)(pair / top) * K;
  const float acc = warp_dot(wr, hr, K, lane);
  float v;
  if (GLU) {
    const float u = warp_dot(wr + up_rows * K, hr, K, lane);
    v = acc / (1.f + expf(-acc)) * u;
  } else {
    v = fmaxf(acc, 0.f);
    v = v * v;
  }
  if (lane == 0) a[(size_t)pair * F + f] = from_f32<T>(v * wts[pair]);
}

// y[t, o] (+)= sum_j W_down[o, e(t, j) F ..] . a[t * top + j]; W_down: [N, ld] (ld columns a row)
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_sparse_kernel(const T* __restrict__ a, const T* __restrict__ w_down, const int* __restrict__ idx,
                       float* __restrict__ y, int store, int top, int F, int ld, int N, int n_real) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (o >= N) return;
  float acc = 0.f;
  for (int j = 0; j < top; ++j) {
    const int e = idx[(size_t)t * top + j];
    if (e >= n_real) continue;
    const T* wr = w_down + (size_t)o * ld + (size_t)e * F;
    const T* ar = a + ((size_t)t * top + j) * F;
    acc += warp_dot(wr, ar, F, lane);
  }
  if (lane == 0) y[(size_t)t * N + o] = store ? acc : y[(size_t)t * N + o] + acc;
}

}  // namespace

CUCA_API int cuca_moe_max_experts() { return MAX_EXPERTS; }

CUCA_API int cuca_moe_route(const float* logits, int T, int E, int top, int* idx, float* wts, float* dense,
                            cudaStream_t stream) {
  if (T == 0) return 0;
  CUCA_REQUIRE(E >= 1 && E <= MAX_EXPERTS && top >= 1 && top <= E && top <= MAX_TOP,
               "moe_route: %d of %d experts is outside what the kernel takes (experts <= %d, chosen <= %d)", top, E,
               MAX_EXPERTS, MAX_TOP);
  cuca_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, true, logits, T, E, top, idx, wts, dense);
  CUCA_CHECK_LAUNCH("moe_route");
  return 0;
}

CUCA_API int cuca_moe_act_dense(const void* u, const float* dense, void* a, int dtype, int T, int E, int F,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  const size_t n = (size_t)T * E * F;
  size_t blocks = (n + 255) / 256;
  blocks = blocks > 8192 ? 8192 : blocks;
  if (dtype == CUCA_F32)
    cuca_launch(moe_act_dense_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, true, (const float*)u, dense,
                (float*)a, n, E, F);
  else if (dtype == CUCA_BF16)
    cuca_launch(moe_act_dense_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, true,
                (const __nv_bfloat16*)u, dense, (__nv_bfloat16*)a, n, E, F);
  else
    CUCA_REQUIRE(false, "moe_act_dense: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("moe_act_dense");
  return 0;
}

// glu 0: relu(up)^2 experts, w_up [E F, K], w_down [N, E F]. glu 1: gated experts, w_up [2 C, K] (every expert's gate
// rows, then C rows on every expert's up rows), w_down [N, C]; C >= E F (what lies behind belongs to a shared expert,
// which this launch leaves alone). Pairs that name expert E or more are skipped.
CUCA_API int cuca_moe_sparse(const void* h, const void* w_up, const void* w_down, const int* idx, const float* wts,
                             void* a, float* y, int store, int dtype, int T, int top, int E, int F, int K, int N,
                             int glu, int C, cudaStream_t stream) {
  if (T == 0) return 0;
  CUCA_REQUIRE(T * top <= 65535 && T <= 65535, "moe_sparse: %d tokens exceed the launch limit", T);
  const int ld = glu ? C : E * F;
  CUCA_REQUIRE(ld >= E * F, "moe_sparse: %d columns do not hold %d experts of %d", ld, E, F);
#define SPARSE(TT)                                                                                                  \
  do {                                                                                                              \
    if (glu)                                                                                                        \
      cuca_launch(moe_up_sparse_kernel<TT, true>, dim3((F + 7) / 8, T * top), dim3(256), 0, stream, true,           \
                  (const TT*)h, (const TT*)w_up, idx, wts, (TT*)a, top, F, K, E, (size_t)C);                        \
    else                                                                                                            \
      cuca_launch(moe_up_sparse_kernel<TT, false>, dim3((F + 7) / 8, T * top), dim3(256), 0, stream, true,          \
                  (const TT*)h, (const TT*)w_up, idx, wts, (TT*)a, top, F, K, E, (size_t)0);                        \
    CUCA_CHECK_LAUNCH("moe_up_sparse");                                                                             \
    cuca_launch(moe_down_sparse_kernel<TT>, dim3((N + 7) / 8, T), dim3(256), 0, stream, true, (const TT*)a,         \
                (const TT*)w_down, idx, y, store, top, F, ld, N, E);                                                \
  } while (0)
  if (dtype == CUCA_F32) SPARSE(float);
  else if (dtype == CUCA_BF16) SPARSE(__nv_bfloat16);
  else CUCA_REQUIRE(false, "moe_sparse: unknown dtype %d", dtype);
#undef SPARSE
  CUCA_CHECK_LAUNCH("moe_down_sparse");
  return 0;
}

CUCA_API int cuca_moe_route_scored(const float* logits, const float* correction, int T, int E, int n_real, int top,
                                   int* idx, float* wts, float* dense, float* ident, cudaStream_t stream) {
  if (T == 0) return 0;
  CUCA_REQUIRE(E >= 1 && E <= MAX_EXPERTS && top >= 1 && top <= E && top <= MAX_TOP && n_real >= 0 && n_real <= E,
               "moe_route: %d of %d experts (%d with weights) is outside what the kernel takes (experts <= %d, "
               "chosen <= %d)", top, E, n_real, MAX_EXPERTS, MAX_TOP);
  cuca_launch(moe_route_scored_kernel, dim3((T + 3) / 4), dim3(128), 0, stream, true, logits, correction, T, E, n_real,
              top, idx, wts, dense, ident);
  CUCA_CHECK_LAUNCH("moe_route_scored");
  return 0;
}

CUCA_API int cuca_moe_glu_dense(const void* gu, const float* dense, int ld_dense, void* a, int dtype, int T, int C,
                                int EF, int F, cudaStream_t stream) {
  if (T == 0) return 0;
  CUCA_REQUIRE(F >= 1 && EF % F == 0 && EF <= C && EF / F <= ld_dense, "moe_glu_dense: bad sizes C=%d EF=%d F=%d", C, EF, F);
  const size_t n = (size_t)T * C;
  const int V = dtype == CUCA_BF16 ? 8 : 4;
  const bool vec = F % V == 0 && EF % V == 0 && C % V == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)a & 15) == 0;
  const size_t work = vec ? n / V : n;
  size_t blocks = (work + 255) / 256;
  blocks = blocks > 16384 ? 16384 : blocks;
  if (dtype == CUCA_F32 && vec)
    cuca_launch(moe_glu_dense_vec_kernel<float, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, true, (const float*)gu,
                dense, ld_dense, (float*)a, work, C, EF, F);
  else if (dtype == CUCA_BF16 && vec)
    cuca_launch(moe_glu_dense_vec_kernel<__nv_bfloat16, 8>, dim3((unsigned)blocks), dim3(256), 0, stream, true,
                (const __nv_bfloat16*)gu, dense, ld_dense, (__nv_bfloat16*)a, work, C, EF, F);
  else if (dtype == CUCA_F32)
    cuca_launch(moe_glu_dense_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, true, (const float*)gu, dense,
                ld_dense, (float*)a, n, C, EF, F);
  else if (dtype == CUCA_BF16)
    cuca_launch(moe_glu_dense_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, true,
                (const __nv_bfloat16*)gu, dense, ld_dense, (__nv_bfloat16*)a, n, C, EF, F);
  else
    CUCA_REQUIRE(false, "moe_glu_dense: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("moe_glu_dense");
  return 0;
}

CUCA_API int cuca_moe_identity_add(float* y, const void* h, int dtype, const float* ident, int store, int T, int N,
                                   cudaStream_t stream) {
  if (T == 0) return 0;
  const size_t n = (size_t)T * N;
  size_t blocks = (n + 255) / 256;
  blocks = blocks > 8192 ? 8192 : blocks;
  if (dtype == CUCA_F32)
    cuca_launch(moe_identity_add_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, true, y, (const float*)h,
                ident, store, n, N);
  else if (dtype == CUCA_BF16)
    cuca_launch(moe_identity_add_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, true, y,
                (const __nv_bfloat16*)h, ident, store, n, N);
  else
    CUCA_REQUIRE(false, "moe_identity_add: unknown dtype %d", dtype);
  CUCA_CHECK_LAUNCH("moe_identity_add");
  return 0;
}
