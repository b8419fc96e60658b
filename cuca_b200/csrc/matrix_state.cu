// Mixers whose per-request state is a matrix per head, S [key channels, value columns], carried in 32-bit:
//   delta_scan      the delta rule with a decay per key channel:
//                     S <- g * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   mlstm_scan      a matrix memory with exponential gates and a running maximum m (0 at the start):
//                     m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise from k alone;
//                     o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)
//   forget_scan     linear attention whose forget gate f (per key channel) is also one minus its write strength:
//                     S <- f * S (rows) + (1 - f) v^T;  o = S^T q
//   retention_scan  linear attention with one fixed decay per head and no denominator:
//                     S <- decay S + k v^T;  o = S^T q
//   head_norm_gate  out = o / rms(o) per head, times a weight (or none), times sigmoid(gate) or silu(gate)
// What does not depend on the state (unit vectors, decays, gates) is computed for all rows at once by a preparing
// kernel, in place. A scan block then takes one (head, request, run of value columns) and walks the request's rows of
// the step in order from the state its slot holds, leaving the new state there. A value column's state rows live in
// the registers of NS neighbouring threads (thread s holds NR consecutive rows); a token's vectors are copied to
// shared memory a few tokens ahead of their use. The arithmetic of a token does not depend on where the sequence was
// cut into steps or chunks; how many threads share a column's sums (and so the order of those sums) depends on how
// many columns the launch has.
#include "common.cuh"
#include <math.h>
#include <stdlib.h>

namespace {

constexpr int MAXR = 32;  // state rows a thread holds at most

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float softplusf_(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float log_sigmoidf_(float v) { return v < 0.f ? v - log1pf(expf(v)) : -log1pf(expf(-v)); }

// sum over the NS neighbouring threads of a value column (NS a power of two, at most 32)
__device__ __forceinline__ float group_sum(float v, int NS) {
  if (NS >= 32) v += __shfl_xor_sync(0xffffffffu, v, 16);
  if (NS >= 16) v += __shfl_xor_sync(0xffffffffu, v, 8);
  if (NS >= 8) v += __shfl_xor_sync(0xffffffffu, v, 4);
  if (NS >= 4) v += __shfl_xor_sync(0xffffffffu, v, 2);
  if (NS >= 2) v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

// An asynchronous copy of 4 or 16 bytes from global to shared memory.
__device__ __forceinline__ void cp_async_f(float* dst, const float* src, bool wide) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  if (wide) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Where key channel r of a staged vector lies in shared memory: thread s of a value column holds the NR consecutive
// channels s NR .. s NR + NR - 1 and reads them 16 bytes at a time; four floats of padding after every NR keep the
// NS threads of a column on different banks.
// (Four channels a thread are 16 bytes a thread: contiguous, nothing to pad.)
template <int NR> __device__ __forceinline__ constexpr int staged_stride() { return NR == 4 ? 4 : NR + 4; }
template <int NR> __device__ __forceinline__ int staged_at(int r) { return (r / NR) * staged_stride<NR>() + r % NR; }

// Per row, in place: q and k heads (G heads of d at columns 0 and G d of qkv) become unit vectors, q times d^(-1/2);
// the decay pre-activations a_raw (rows of stride ld_a, H d values) become g = exp(-exp(A_log[h]) softplus(a + dt_bias)); the gate
// pre-activation of head h (column b_col + h of b_raw) becomes sigmoid. One block per row.
__global__ void __launch_bounds__(256)
delta_prepare_kernel(float* __restrict__ qkv, int ld, float* __restrict__ a_raw, int ld_a, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, float* __restrict__ b_raw, int ld_b, int b_col,
                     const int* __restrict__ seq_of_row, int H, int G, int d) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  if (seq_of_row[row] < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float qscale = rsqrtf((float)d);
  for (int v = warp; v < 2 * G; v += 8) {  // q heads, then k heads
    float* x = qkv + row * ld + (size_t)v * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss = fmaf(x[i], x[i], ss);
    const float inv = (v < G ? qscale : 1.f) / sqrtf(warp_sum(ss) + 1e-6f);
    for (int i = lane; i < d; i += 32) x[i] *= inv;
  }
  float* ar = a_raw + row * ld_a;
  for (int i = threadIdx.x; i < H * d; i += 256)
    ar[i] = expf(-expf(a_log[i / d]) * softplusf_(ar[i] + dt_bias[i]));
  if (threadIdx.x < H) {
    float* b = b_raw + row * ld_b + b_col + threadIdx.x;
    *b = sigmoidf_(*b);
  }
}

// qkv: 32-bit rows of stride ld, prepared: unit q heads at column 0 (G heads of d), unit k heads at column G d, v
// heads at column 2 G d (H heads of dv). g: rows of stride ld_g, H d decays; beta: rows of stride ld_b, head h at column
// b_col + h. state: [slots, H, dv, d]. out: [rows, H dv]. Two buffers of TC tokens: the next tokens' vectors are
// copied (cp.async) while these are worked through.
template <int NR>
__global__ void delta_scan_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ g, int ld_g,
                                  const float* __restrict__ beta, int ld_b, int b_col, float* __restrict__ state,
                                  float* __restrict__ out, const int* __restrict__ req_row0,
                                  const int* __restrict__ req_count, const int* __restrict__ slots, int H, int G,
                                  int d, int dv, int NS, int PB, int TC, int wide) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, rq = blockIdx.y;
  const int slot = slots[rq], n = req_count[rq], r0 = req_row0[rq];
  if (slot < 0 || n <= 0) return;
  const int kvh = h / (H / G);
  const int dpp = NS * staged_stride<NR>();     // a staged vector with its padding
  const int per = (3 * dpp + PB + 1 + 3) & ~3;  // a token: q, k, g, the block's values, beta
  const int col_local = threadIdx.x / NS, s = threadIdx.x % NS;
  const int col = blockIdx.z * PB + col_local;
  const bool live = col_local < PB && col < dv;
  float S[NR];
  float* st = state + (((size_t)slot * H + h) * dv + (live ? col : 0)) * d;
#pragma unroll
  for (int i = 0; i < NR; ++i) S[i] = (live && s * NR + i < d) ? st[s * NR + i] : 0.f;
  // what no copy writes: channels from d on (q = k = 0, g = 1) and the values of columns from dv on
  {
    const int spare = NS * NR - d, fill = 3 * spare + PB;
    for (int e = threadIdx.x; e < 2 * TC * fill; e += blockDim.x) {
      const int t = e / fill, w = e % fill;
      float* tok = sm + (size_t)t * per;
      if (w < 3 * spare) tok[(w / spare) * dpp + staged_at<NR>(d + w % spare)] = w / spare == 2 ? 1.f : 0.f;
      else tok[3 * dpp + (w - 3 * spare)] = 0.f;
    }
  }
  __syncthreads();
  auto stage = [&](int t0, int buf) {
    const int nt = n - t0 < TC ? n - t0 : TC;
    float* base = sm + (size_t)buf * TC * per;
    const int step = wide ? 4 : 1, units = d / step;
    for (int e = threadIdx.x; e < nt * 3 * units; e += blockDim.x) {
      const int t = e / (3 * units), u = e % (3 * units), which = u / units, r = (u % units) * step;
      const size_t row = (size_t)(r0 + t0 + t);
      const float* src = which == 0 ? qkv + row * ld + (size_t)kvh * d + r
                       : which == 1 ? qkv + row * ld + (size_t)(G + kvh) * d + r
                                    : g + row * ld_g + (size_t)h * d + r;
      cp_async_f(base + (size_t)t * per + which * dpp + staged_at<NR>(r), src, wide);
    }
    for (int e = threadIdx.x; e < nt * (PB + 1); e += blockDim.x) {
      const int t = e / (PB + 1), i = e % (PB + 1);
      const size_t row = (size_t)(r0 + t0 + t);
      if (i == PB) cp_async_f(base + (size_t)t * per + 3 * dpp + PB, beta + row * ld_b + b_col + h, false);
      else if (blockIdx.z * PB + i < dv)
        cp_async_f(base + (size_t)t * per + 3 * dpp + i, qkv + row * ld + (size_t)2 * G * d + (size_t)h * dv + blockIdx.z * PB + i, false);
    }
    cp_async_commit();
  };
  const int cv = col_local < PB ? col_local : PB - 1;
  const int n_chunks = (n + TC - 1) / TC;
  stage(0, 0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) { stage((c + 1) * TC, (c + 1) & 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int t0 = c * TC, nt = n - t0 < TC ? n - t0 : TC;
    const float* base = sm + (size_t)(c & 1) * TC * per;
    // every thread of a warp takes part (the sums shuffle across whole warps); spare threads work on zeros
    const float* tok = base;
    float* po_at = out + (size_t)(r0 + t0) * H * dv + (size_t)h * dv + col;
    const int mine = s * staged_stride<NR>(), extra = 3 * dpp;
#pragma unroll 2
    for (int t = 0; t < nt; ++t, tok += per, po_at += H * dv) {
      const float4* gq = reinterpret_cast<const float4*>(tok + mine);
      const float4* gk = reinterpret_cast<const float4*>(tok + dpp + mine);
      const float4* gg = reinterpret_cast<const float4*>(tok + 2 * dpp + mine);
      float kk[NR];
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int i = 0; i < NR / 4; ++i) {
        const float4 gv = gg[i], kv4 = gk[i];
        kk[4 * i] = kv4.x; kk[4 * i + 1] = kv4.y; kk[4 * i + 2] = kv4.z; kk[4 * i + 3] = kv4.w;
        S[4 * i] *= gv.x; S[4 * i + 1] *= gv.y; S[4 * i + 2] *= gv.z; S[4 * i + 3] *= gv.w;
        p0 = fmaf(S[4 * i], kv4.x, p0); p1 = fmaf(S[4 * i + 1], kv4.y, p1);
        p2 = fmaf(S[4 * i + 2], kv4.z, p2); p3 = fmaf(S[4 * i + 3], kv4.w, p3);
      }
      const float part = group_sum((p0 + p1) + (p2 + p3), NS);
      const float u = tok[extra + PB] * (tok[extra + cv] - part);
      p0 = p1 = p2 = p3 = 0.f;
#pragma unroll
      for (int i = 0; i < NR / 4; ++i) {
        const float4 qv = gq[i];
        S[4 * i] = fmaf(kk[4 * i], u, S[4 * i]); S[4 * i + 1] = fmaf(kk[4 * i + 1], u, S[4 * i + 1]);
        S[4 * i + 2] = fmaf(kk[4 * i + 2], u, S[4 * i + 2]); S[4 * i + 3] = fmaf(kk[4 * i + 3], u, S[4 * i + 3]);
        p0 = fmaf(S[4 * i], qv.x, p0); p1 = fmaf(S[4 * i + 1], qv.y, p1);
        p2 = fmaf(S[4 * i + 2], qv.z, p2); p3 = fmaf(S[4 * i + 3], qv.w, p3);
      }
      const float po = group_sum((p0 + p1) + (p2 + p3), NS);
      if (s == 0 && live) *po_at = po;
    }
    __syncthreads();  // the buffer is free for the copies of the chunk after next
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (s * NR + i < d) st[s * NR + i] = S[i];
  }
}

// Per row, in place, of a 32-bit projection [q | f | ...]: q (H d values at q_col) becomes silu(q); the forget gate's
// pre-activation (H d values at f_col) becomes f = l + (1 - l) sigmoid(x + bias) with a lower bound l per channel.
__global__ void forget_prepare_kernel(float* __restrict__ proj, int ld, int q_col, int f_col,
                                      const float* __restrict__ f_bias, const float* __restrict__ lower,
                                      const int* __restrict__ seq_of_row, int n_rows, int n) {
  pdl_trigger();
  pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < (size_t)n_rows * n; e += (size_t)gridDim.x * blockDim.x) {
    const size_t row = e / n;
    const int i = (int)(e % n);
    if (seq_of_row[row] < 0) continue;
    float* r = proj + row * ld;
    const float q = r[q_col + i];
    r[q_col + i] = q * sigmoidf_(q);
    const float l = lower[i];
    r[f_col + i] = l + (1.f - l) * sigmoidf_(r[f_col + i] + (f_bias ? f_bias[i] : 0.f));
  }
}

// Per row, in place, of a 32-bit projection [q | k | ...] (H heads of d each): the first `rot` values of every q and k
// head turn by the row's position in pairs (i, i + rot/2) with the angle tables' row of that position; k is then
// multiplied by k_scale. One thread per (row, head, pair or unrotated value).
__global__ void retention_prepare_kernel(float* __restrict__ proj, int ld, int q_col, int k_col,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         int table_rows, int rot, float k_scale, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_row, int n_rows, int H, int d, int* err) {
  pdl_trigger();
  pdl_wait();
  const int half = rot / 2, per_head = half + (d - rot);
  const size_t per_row = (size_t)2 * H * per_head;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < (size_t)n_rows * per_row;
       e += (size_t)gridDim.x * blockDim.x) {
    const size_t row = e / per_row;
    const int w = (int)(e % per_row);
    if (seq_of_row[row] < 0) continue;
    const int which = w / (H * per_head), hh = (w / per_head) % H, i = w % per_head;
    float* head = proj + row * ld + (which ? k_col : q_col) + (size_t)hh * d;
    const float mul = which ? k_scale : 1.f;
    if (i < half) {
      const int pos = positions[row];
      if (pos < 0 || pos >= table_rows) {
        if (err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
        continue;
      }
      const float c = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
      const float a = head[i], b = head[i + half];
      head[i] = (a * c - b * sn) * mul;
      head[i + half] = (b * c + a * sn) * mul;
    } else if (which) {
      head[rot + (i - half)] *= mul;
    }
  }
}

// proj: 32-bit rows of stride ld, prepared: q heads at q_col (H heads of d), forget gates at f_col (H heads of d),
// v heads at v_col (H heads of dv). state: [slots, H, dv, d]. out: [rows, H dv]. The delta scan's sibling without a
// correction: one shuffled sum per token and column.
// RET (retention): the second staged vector is the key k instead of the gate, and the state decays by one number per
// head: S <- decay[h] S + k v^T.
template <int NR, bool RET>
__global__ void forget_scan_kernel(const float* __restrict__ proj, int ld, int q_col, int f_col, int v_col,
                                   const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out,
                                   const int* __restrict__ req_row0, const int* __restrict__ req_count,
                                   const int* __restrict__ slots, int H, int d, int dv, int NS, int PB, int TC, int wide) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, rq = blockIdx.y;
  const int slot = slots[rq], n = req_count[rq], r0 = req_row0[rq];
  if (slot < 0 || n <= 0) return;
  const int dpp = NS * staged_stride<NR>();  // a staged vector with its padding
  const int per = (2 * dpp + PB + 3) & ~3;   // a token: q, f, the block's values
  const int col_local = threadIdx.x / NS, s = threadIdx.x % NS;
  const int col = blockIdx.z * PB + col_local;
  const bool live = col_local < PB && col < dv;
  float S[NR];
  float* st = state + (((size_t)slot * H + h) * dv + (live ? col : 0)) * d;
#pragma unroll
  for (int i = 0; i < NR; ++i) S[i] = (live && s * NR + i < d) ? st[s * NR + i] : 0.f;
  // what no copy writes: channels from d on (q = 0, f = 1) and the values of columns from dv on
  {
    const int spare = NS * NR - d, fill = 2 * spare + PB;
    for (int e = threadIdx.x; e < 2 * TC * fill; e += blockDim.x) {
      const int t = e / fill, w = e % fill;
      float* tok = sm + (size_t)t * per;
      if (w < 2 * spare) tok[(w / spare) * dpp + staged_at<NR>(d + w % spare)] = (w / spare == 1 && !RET) ? 1.f : 0.f;
      else tok[2 * dpp + (w - 2 * spare)] = 0.f;
    }
  }
  __syncthreads();
  auto stage = [&](int t0, int buf) {
    const int nt = n - t0 < TC ? n - t0 : TC;
    float* base = sm + (size_t)buf * TC * per;
    const int step = wide ? 4 : 1, units = d / step;
    for (int e = threadIdx.x; e < nt * 2 * units; e += blockDim.x) {
      const int t = e / (2 * units), u = e % (2 * units), which = u / units, r = (u % units) * step;
      const float* src = proj + (size_t)(r0 + t0 + t) * ld + (which ? f_col : q_col) + (size_t)h * d + r;
      cp_async_f(base + (size_t)t * per + which * dpp + staged_at<NR>(r), src, wide);
    }
    for (int e = threadIdx.x; e < nt * PB; e += blockDim.x) {
      const int t = e / PB, i = e % PB;
      if (blockIdx.z * PB + i < dv)
        cp_async_f(base + (size_t)t * per + 2 * dpp + i,
                   proj + (size_t)(r0 + t0 + t) * ld + v_col + (size_t)h * dv + blockIdx.z * PB + i, false);
    }
    cp_async_commit();
  };
  const int cv = col_local < PB ? col_local : PB - 1;
  const int n_chunks = (n + TC - 1) / TC;
  const float dec = RET ? decay[h] : 0.f;
  stage(0, 0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) { stage((c + 1) * TC, (c + 1) & 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int t0 = c * TC, nt = n - t0 < TC ? n - t0 : TC;
    const float* tok = sm + (size_t)(c & 1) * TC * per;
    float* po_at = out + (size_t)(r0 + t0) * H * dv + (size_t)h * dv + col;
    const int mine = s * staged_stride<NR>();
    // (tokens depend on each other through the state's one multiply-add alone: with four rows a thread, eight
    // tokens in flight keep the loads and the shuffled sums of the next ones going while these wait)
#pragma unroll(NR == 4 ? 8 : 2)
    for (int t = 0; t < nt; ++t, tok += per, po_at += H * dv) {
      const float4* gq = reinterpret_cast<const float4*>(tok + mine);
      const float4* gf = reinterpret_cast<const float4*>(tok + dpp + mine);
      const float v = tok[2 * dpp + cv];
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int i = 0; i < NR / 4; ++i) {
        const float4 f4 = gf[i], qv = gq[i];
        if (RET) {  // decay S + k v
          S[4 * i] = fmaf(dec, S[4 * i], f4.x * v); S[4 * i + 1] = fmaf(dec, S[4 * i + 1], f4.y * v);
          S[4 * i + 2] = fmaf(dec, S[4 * i + 2], f4.z * v); S[4 * i + 3] = fmaf(dec, S[4 * i + 3], f4.w * v);
        } else {
        // f S + (1 - f) v, each product rounded as the plain recurrence rounds it
        S[4 * i] = fmaf(f4.x, S[4 * i], (1.f - f4.x) * v); S[4 * i + 1] = fmaf(f4.y, S[4 * i + 1], (1.f - f4.y) * v);
        S[4 * i + 2] = fmaf(f4.z, S[4 * i + 2], (1.f - f4.z) * v); S[4 * i + 3] = fmaf(f4.w, S[4 * i + 3], (1.f - f4.w) * v);
        }
        p0 = fmaf(S[4 * i], qv.x, p0); p1 = fmaf(S[4 * i + 1], qv.y, p1);
        p2 = fmaf(S[4 * i + 2], qv.z, p2); p3 = fmaf(S[4 * i + 3], qv.w, p3);
      }
      const float po = group_sum((p0 + p1) + (p2 + p3), NS);
      if (s == 0 && live) *po_at = po;
    }
    __syncthreads();  // the buffer is free for the copies of the chunk after next
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (s * NR + i < d) st[s * NR + i] = S[i];
  }
}

// Per row, in place: the raw input gate of head h (column i_col + h of proj) becomes cap tanh((x + b_i) / cap), the
// raw forget gate (column f_col + h) becomes logsigmoid(cap tanh((x + b_f) / cap)).
__global__ void mlstm_prepare_kernel(float* __restrict__ proj, int ld, int i_col, int f_col,
                                     const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                                     int n_rows, int H) {
  pdl_trigger();
  pdl_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_rows * H) return;
  float* row = proj + (size_t)(e / H) * ld;
  const int h = e % H;
  row[i_col + h] = cap * tanhf((row[i_col + h] + (i_bias ? i_bias[h] : 0.f)) / cap);
  row[f_col + h] = log_sigmoidf_(cap * tanhf((row[f_col + h] + (f_bias ? f_bias[h] : 0.f)) / cap));
}

// proj: 32-bit rows of stride ld, prepared: q heads at q_col (H heads of d), k at k_col, v at v_col (H heads of dv),
// the log input gate of head h at i_col + h, the log forget gate at f_col + h.
// mem: [slots, H, dv, d]; nrm: [slots, H, d]; mx: [slots, H]. out: [rows, H dv].
// The block's columns are its PB value columns and one more that carries n (its "value" is 1), so n . q comes out
// of the same loop; the division waits until the chunk's sums are in shared memory. q enters unscaled: the sums
// are linear in it, so d^(-1/2) multiplies them afterwards. n and m are shared by all blocks of a (head, request):
// this launch only reads them and leaves the new ones aside (nm_new); `mlstm_commit_kernel` moves them into the slots.
template <int NR>
__global__ void mlstm_scan_kernel(const float* __restrict__ proj, int ld, int q_col, int k_col, int v_col, int i_col,
                                  int f_col, float* __restrict__ mem, float* __restrict__ nrm, float* __restrict__ mx,
                                  float* __restrict__ out, const int* __restrict__ req_row0,
                                  const int* __restrict__ req_count, const int* __restrict__ slots, int H, int d,
                                  int dv, int NS, int PB, int TC, int wide, float* __restrict__ nm_new) {
  extern __shared__ __align__(16) float sm[];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, rq = blockIdx.y;
  const int slot = slots[rq], n = req_count[rq], r0 = req_row0[rq];
  if (slot < 0 || n <= 0) return;
  const int dpp = NS * staged_stride<NR>();
  const int per = (2 * dpp + (PB + 1) + 2 + 3) & ~3;  // a token: q, k, the block's values and a 1, the two gates
  float* so = sm + (size_t)2 * TC * per;     // [TC][PB + 1] the chunk's sums
  float* keep = so + (size_t)TC * (PB + 1);  // [TC] e^(f + m - m')
  float* take = keep + TC;                   // [TC] e^(i - m')
  float* floor_ = take + TC;                 // [TC] e^(-m')
  float* ms = floor_ + TC;                   // [TC + 1] m before each token of the chunk, and after the last
  const int col_local = threadIdx.x / NS, s = threadIdx.x % NS;
  const bool is_n = col_local == PB;
  const int col = blockIdx.z * PB + col_local;
  const bool live = is_n || (col_local < PB && col < dv);
  float S[NR];
  float* st = is_n ? nrm + ((size_t)slot * H + h) * d
                   : mem + (((size_t)slot * H + h) * dv + (col < dv ? col : 0)) * d;
#pragma unroll
  for (int i = 0; i < NR; ++i) S[i] = (live && s * NR + i < d) ? st[s * NR + i] : 0.f;
  {
    const int spare = NS * NR - d, fill = 2 * spare + PB + 1;
    for (int e = threadIdx.x; e < 2 * TC * fill; e += blockDim.x) {
      const int t = e / fill, w = e % fill;
      float* tok = sm + (size_t)t * per;
      if (w < 2 * spare) tok[(w / spare) * dpp + staged_at<NR>(d + w % spare)] = 0.f;
      else tok[2 * dpp + (w - 2 * spare)] = w - 2 * spare == PB ? 1.f : 0.f;
    }
  }
  if (threadIdx.x == 0) ms[0] = mx[(size_t)slot * H + h];
  __syncthreads();
  const float qscale = rsqrtf((float)d);
  auto stage = [&](int t0, int buf) {
    const int nt = n - t0 < TC ? n - t0 : TC;
    float* base = sm + (size_t)buf * TC * per;
    const int step = wide ? 4 : 1, units = d / step;
    for (int e = threadIdx.x; e < nt * 2 * units; e += blockDim.x) {
      const int t = e / (2 * units), u = e % (2 * units), which = u / units, r = (u % units) * step;
      const float* src = proj + (size_t)(r0 + t0 + t) * ld + (which ? k_col : q_col) + (size_t)h * d + r;
      cp_async_f(base + (size_t)t * per + which * dpp + staged_at<NR>(r), src, wide);
    }
    for (int e = threadIdx.x; e < nt * (PB + 2); e += blockDim.x) {
      const int t = e / (PB + 2), i = e % (PB + 2);
      const float* row = proj + (size_t)(r0 + t0 + t) * ld;
      float* tok = base + (size_t)t * per + 2 * dpp;
      if (i == PB) cp_async_f(tok + PB + 1, row + i_col + h, false);
      else if (i == PB + 1) cp_async_f(tok + PB + 2, row + f_col + h, false);
      else if (blockIdx.z * PB + i < dv) cp_async_f(tok + i, row + v_col + (size_t)h * dv + blockIdx.z * PB + i, false);
    }
    cp_async_commit();
  };
  const int cv = col_local <= PB ? col_local : PB;
  const int n_chunks = (n + TC - 1) / TC;
  stage(0, 0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c + 1 < n_chunks) { stage((c + 1) * TC, (c + 1) & 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int t0 = c * TC, nt = n - t0 < TC ? n - t0 : TC;
    const float* base = sm + (size_t)(c & 1) * TC * per;
    if (threadIdx.x == 0) {  // the running maximum is a chain of one add and one max per token
      float m = ms[0];
      for (int t = 0; t < nt; ++t) {
        const float* tok = base + (size_t)t * per + 2 * dpp;
        m = fmaxf(tok[PB + 2] + m, tok[PB + 1]);
        ms[t + 1] = m;
      }
    }
    __syncthreads();
    if (threadIdx.x < nt) {
      const int t = threadIdx.x;
      const float* tok = base + (size_t)t * per + 2 * dpp;
      keep[t] = expf(tok[PB + 2] + ms[t] - ms[t + 1]);
      take[t] = expf(tok[PB + 1] - ms[t + 1]);
      floor_[t] = expf(-ms[t + 1]);
    }
    __syncthreads();
    const float* tok = base;
    const int mine = s * staged_stride<NR>();
    float* so_at = so + col_local;
#pragma unroll 2
    for (int t = 0; t < nt; ++t, tok += per, so_at += PB + 1) {
      const float4* gq = reinterpret_cast<const float4*>(tok + mine);
      const float4* gk = reinterpret_cast<const float4*>(tok + dpp + mine);
      const float kp = keep[t], w = take[t] * tok[2 * dpp + cv];
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int i = 0; i < NR / 4; ++i) {
        const float4 kv4 = gk[i], qv = gq[i];
        S[4 * i] = fmaf(kp, S[4 * i], w * kv4.x); S[4 * i + 1] = fmaf(kp, S[4 * i + 1], w * kv4.y);
        S[4 * i + 2] = fmaf(kp, S[4 * i + 2], w * kv4.z); S[4 * i + 3] = fmaf(kp, S[4 * i + 3], w * kv4.w);
        p0 = fmaf(S[4 * i], qv.x, p0); p1 = fmaf(S[4 * i + 1], qv.y, p1);
        p2 = fmaf(S[4 * i + 2], qv.z, p2); p3 = fmaf(S[4 * i + 3], qv.w, p3);
      }
      const float po = group_sum((p0 + p1) + (p2 + p3), NS) * qscale;
      if (s == 0 && col_local <= PB) *so_at = po;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * PB; e += blockDim.x) {
      const int t = e / PB, i = e % PB;
      if (blockIdx.z * PB + i < dv) {
        const float den = fmaxf(fabsf(so[(size_t)t * (PB + 1) + PB]), floor_[t]) + 1e-6f;
        out[(size_t)(r0 + t0 + t) * H * dv + (size_t)h * dv + blockIdx.z * PB + i] = so[(size_t)t * (PB + 1) + i] / den;
      }
    }
    if (threadIdx.x == 0) ms[0] = ms[nt];
    __syncthreads();  // the buffers and the chunk's sums are free again
  }
  // every block of a (head, request) starts from the same n and m, so no block of this launch may replace them:
  // the block of the first columns leaves the new ones in nm_new [requests, H, d + 1], and a launch of its own
  // moves them into the slots once this one is through
  if (live && col_local < PB) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (s * NR + i < d) st[s * NR + i] = S[i];
  }
  float* nm = nm_new + ((size_t)rq * H + h) * (d + 1);
  if (is_n && blockIdx.z == 0) {
#pragma unroll
    for (int i = 0; i < NR; ++i)
      if (s * NR + i < d) nm[s * NR + i] = S[i];
  }
  if (threadIdx.x == 0 && blockIdx.z == 0) nm[d] = ms[0];
}

__global__ void mlstm_commit_kernel(const float* __restrict__ nm_new, float* __restrict__ nrm, float* __restrict__ mx,
                                    const int* __restrict__ req_count, const int* __restrict__ slots, int H, int d) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, rq = blockIdx.y;
  const int slot = slots[rq];
  if (slot < 0 || req_count[rq] <= 0) return;
  const float* nm = nm_new + ((size_t)rq * H + h) * (d + 1);
  for (int i = threadIdx.x; i < d; i += blockDim.x) nrm[((size_t)slot * H + h) * d + i] = nm[i];
  if (threadIdx.x == 0) mx[(size_t)slot * H + h] = nm[d];
}

// o: [rows, H dv] 32-bit. out[r, h, j] = o / sqrt(mean_j o^2 + eps) * w[h * w_head + j] * sigmoid(gate[r, h dv + j]);
// w_head 0: one weight vector for every head; w null: no weight. gate: rows of stride ld_g (TG), null for none;
// SILU: the gate's factor is silu(gate) instead of sigmoid(gate).
template <typename TG, typename TO, bool SILU>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_head,
                      const TG* __restrict__ gate, int ld_g, TO* __restrict__ out, int H, int dv, float eps,
                      long long n_items) {
  pdl_trigger();
  pdl_wait();
  // a warp per (row, head); 16 bytes of o a lane at a time where a head's values allow it
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_items) return;
  const size_t row = (size_t)(item / H);
  const int h = (int)(item % H);
  const float* orow = o + (size_t)item * dv;
  const float* wh = w ? w + (size_t)h * w_head : nullptr;
  auto gate_of = [](float g) { return SILU ? g * sigmoidf_(g) : sigmoidf_(g); };
  const TG* grow = gate ? gate + row * ld_g + (size_t)h * dv : nullptr;
  TO* dst = out + (size_t)item * dv;
  if ((dv & 3) == 0) {
    float ss = 0.f;
    for (int j = lane * 4; j < dv; j += 128) {
      const float4 v = *reinterpret_cast<const float4*>(orow + j);
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int j = lane * 4; j < dv; j += 128) {
      const float4 v = *reinterpret_cast<const float4*>(orow + j);
      float r[4] = {v.x * inv, v.y * inv, v.z * inv, v.w * inv};
      if (wh) {
#pragma unroll
        for (int e = 0; e < 4; ++e) r[e] *= wh[j + e];
      }
      if (grow) {
#pragma unroll
        for (int e = 0; e < 4; ++e) r[e] *= gate_of(to_f32(grow[j + e]));
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) dst[j + e] = from_f32<TO>(r[e]);
    }
    return;
  }
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(orow[j], orow[j], ss);
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int j = lane; j < dv; j += 32) {
    float v = orow[j] * inv * (wh ? wh[j] : 1.f);
    if (grow) v *= gate_of(to_f32(grow[j]));
    dst[j] = from_f32<TO>(v);
  }
}

int round_nr(int nr) { return nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32; }

// (threads per value column, state rows per thread) for d key channels and `columns` value columns in the whole
// launch. A column's chain of arithmetic per token is serial, so a launch with few columns (one prompt) is bound by
// latency: it gets more threads per column, down to four state rows each, until the GPU's schedulers have several
// warps apiece; a launch with many columns (a batch of single tokens) keeps longer rows per thread.
bool split_rows(int d, long long columns, int* ns_out, int* nr_out) {
  int ns = 1;
  while ((d + ns - 1) / ns > MAXR && ns < 32) ns <<= 1;
  if ((d + ns - 1) / ns > MAXR) return false;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  static const int forced = getenv("CUCA_SCAN_THREADS") ? atoi(getenv("CUCA_SCAN_THREADS")) : 0;  // a measuring aid
  while (ns < 32 && ns * 4 <= d && (forced ? ns < forced : columns * ns < (long long)sms * 2048)) ns <<= 1;
  *ns_out = ns;
  *nr_out = round_nr((d + ns - 1) / ns);
  return true;
}

// threads of a block: 512 where a column has 16 threads or more (the block's staged vectors then serve more
// columns), else 128. Measured on 2,048-token prompts, 32 threads a column: at 16 heads of 128 x 128 blocks of 128
// threads are 5 % faster for the whole prompt step than blocks of 512 (15.9 against 16.9 ms), at 24 and 32 heads they
// are 17 % slower (23.7 against 20.1 ms, 28.9 against 24.7): 512 stays.
int block_threads(int ns, int nr) {
  static const int forced = getenv("CUCA_SCAN_BLOCK") ? atoi(getenv("CUCA_SCAN_BLOCK")) : 0;  // a measuring aid
  if (forced >= ns && forced <= 512) return forced;
  return ns >= 16 ? (nr >= 16 ? 256 : 512) : 128;
}

}  // namespace

CUCA_API int cuca_matrix_state_max_dim() { return 32 * MAXR; }

// qkv, a_raw and the gate column of b_raw are rewritten in place by the preparing kernel (see there), then scanned.
CUCA_API int cuca_delta_scan(float* qkv, int ld, float* a_raw, int ld_a, const float* dt_bias, const float* a_log,
                             float* b_raw, int ld_b, int b_col, float* state, float* out, const int* seq_of_row,
                             const int* req_row0, const int* req_count, const int* slots, int n_rows, int n_seqs, int H,
                             int G, int d, int dv, cudaStream_t stream) {
  if (n_seqs == 0 || n_rows == 0) return 0;
  CUCA_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0, "delta_scan: bad sizes heads=%d key heads=%d dim=%d vdim=%d",
               H, G, d, dv);
  CUCA_REQUIRE(n_seqs <= 65535 && H <= 256, "delta_scan: %d requests or %d heads exceed the launch limits", n_seqs, H);
  int ns, nr;
  CUCA_REQUIRE(split_rows(d, (long long)n_seqs * H * dv, &ns, &nr), "delta_scan: %d key channels exceed %d", d, 32 * MAXR);
  cuca_launch(delta_prepare_kernel, dim3(n_rows), dim3(256), 0, stream, true, qkv, ld, a_raw, ld_a, dt_bias, a_log, b_raw, ld_b,
              b_col, seq_of_row, H, G, d);
  CUCA_CHECK_LAUNCH("delta_prepare");
  int pb = block_threads(ns, nr) / ns;
  pb = pb > dv ? dv : pb;
  const int threads = (pb * ns + 31) / 32 * 32;
  const int per = (3 * ns * (nr == 4 ? 4 : nr + 4) + pb + 1 + 3) & ~3;
  int tc = 46000 / (2 * per * 4);
  tc = tc > 16 ? 16 : tc;
  CUCA_REQUIRE(tc >= 1, "delta_scan: a token of %d key channels does not fit shared memory", d);
  const size_t smem = (size_t)2 * tc * per * 4;
  // 16-byte copies where every source is aligned for them
  const int wide = d % 4 == 0 && ld % 4 == 0 && ld_a % 4 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)a_raw & 15) == 0;
  dim3 grid(H, n_seqs, (dv + pb - 1) / pb);
#define DS(NR)                                                                                                    \
  cuca_launch(delta_scan_kernel<NR>, grid, dim3(threads), smem, stream, true, (const float*)qkv, ld,              \
              (const float*)a_raw, ld_a, (const float*)b_raw, ld_b, b_col, state, out, req_row0, req_count, slots, H, G, d, \
              dv, ns, pb, tc, wide)
  if (nr == 4) DS(4);
  else if (nr == 8) DS(8);
  else if (nr == 16) DS(16);
  else DS(32);
#undef DS
  CUCA_CHECK_LAUNCH("delta_scan");
  return 0;
}

// The two gate columns of proj are rewritten in place by the preparing kernel (see there), then scanned.
// nm_new: scratch of n_seqs * H * (d + 1) floats.
CUCA_API int cuca_mlstm_scan(float* proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float* mem, float* nrm, float* mx,
                             float* out, float* nm_new, const int* req_row0, const int* req_count, const int* slots,
                             int n_rows, int n_seqs, int H, int d, int dv, cudaStream_t stream) {
  if (n_seqs == 0 || n_rows == 0) return 0;
  CUCA_REQUIRE(H > 0 && d > 0 && dv > 0 && cap > 0.f, "mlstm_scan: bad sizes heads=%d dim=%d vdim=%d cap=%g", H, d, dv,
               (double)cap);
  CUCA_REQUIRE(n_seqs <= 65535, "mlstm_scan: %d requests exceed the launch limit", n_seqs);
  int ns, nr;
  CUCA_REQUIRE(split_rows(d, (long long)n_seqs * H * dv, &ns, &nr), "mlstm_scan: %d key channels exceed %d", d, 32 * MAXR);
  cuca_launch(mlstm_prepare_kernel, dim3((n_rows * H + 127) / 128), dim3(128), 0, stream, true, proj, ld, i_col, f_col,
              i_bias, f_bias, cap, n_rows, H);
  CUCA_CHECK_LAUNCH("mlstm_prepare");
  int pb = block_threads(ns, nr) / ns - 1;  // one more column carries n
  pb = pb < 1 ? 1 : (pb > dv ? dv : pb);
  const int threads = ((pb + 1) * ns + 31) / 32 * 32;
  const int per = (2 * ns * (nr == 4 ? 4 : nr + 4) + (pb + 1) + 2 + 3) & ~3;
  int tc = 46000 / ((2 * per + pb + 6) * 4);
  tc = tc > 16 ? 16 : tc;
  CUCA_REQUIRE(tc >= 1, "mlstm_scan: a token of %d key channels does not fit shared memory", d);
  const size_t smem = ((size_t)2 * tc * per + (size_t)tc * (pb + 1) + 4 * tc + 1) * 4;
  const int wide = d % 4 == 0 && ld % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0 && ((uintptr_t)proj & 15) == 0;
  dim3 grid(H, n_seqs, (dv + pb - 1) / pb);
#define MS(NR)                                                                                                      \
  cuca_launch(mlstm_scan_kernel<NR>, grid, dim3(threads), smem, stream, true, (const float*)proj, ld, q_col, k_col,   \
              v_col, i_col, f_col, mem, nrm, mx, out, req_row0, req_count, slots, H, d, dv, ns, pb, tc, wide, nm_new)
  if (nr == 4) MS(4);
  else if (nr == 8) MS(8);
  else if (nr == 16) MS(16);
  else MS(32);
#undef MS
  CUCA_CHECK_LAUNCH("mlstm_scan");
  cuca_launch(mlstm_commit_kernel, dim3(H, n_seqs), dim3(128), 0, stream, true, (const float*)nm_new, nrm, mx, req_count,
              slots, H, d);
  CUCA_CHECK_LAUNCH("mlstm_commit");
  return 0;
}

// The q and forget-gate columns of proj are rewritten in place by the preparing kernel (see there), then scanned.
CUCA_API int cuca_forget_scan(float* proj, int ld, int q_col, int f_col, int v_col, const float* f_bias,
                              const float* lower, float* state, float* out, const int* seq_of_row, const int* req_row0,
                              const int* req_count, const int* slots, int n_rows, int n_seqs, int H, int d, int dv,
                              cudaStream_t stream) {
  if (n_seqs == 0 || n_rows == 0) return 0;
  CUCA_REQUIRE(H > 0 && d > 0 && dv > 0, "forget_scan: bad sizes heads=%d dim=%d vdim=%d", H, d, dv);
  CUCA_REQUIRE(n_seqs <= 65535, "forget_scan: %d requests exceed the launch limit", n_seqs);
  int ns, nr;
  CUCA_REQUIRE(split_rows(d, (long long)n_seqs * H * dv, &ns, &nr), "forget_scan: %d key channels exceed %d", d, 32 * MAXR);
  {
    size_t blocks = ((size_t)n_rows * H * d + 255) / 256;
    blocks = blocks > 8192 ? 8192 : blocks;
    cuca_launch(forget_prepare_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, true, proj, ld, q_col, f_col, f_bias,
                lower, seq_of_row, n_rows, H * d);
    CUCA_CHECK_LAUNCH("forget_prepare");
  }
  int pb = block_threads(ns, nr) / ns;
  pb = pb > dv ? dv : pb;
  const int threads = (pb * ns + 31) / 32 * 32;
  const int per = (2 * ns * (nr == 4 ? 4 : nr + 4) + pb + 3) & ~3;
  int tc = 46000 / (2 * per * 4);
  tc = tc > 16 ? 16 : tc;
  CUCA_REQUIRE(tc >= 1, "forget_scan: a token of %d key channels does not fit shared memory", d);
  const size_t smem = (size_t)2 * tc * per * 4;
  const int wide = d % 4 == 0 && ld % 4 == 0 && q_col % 4 == 0 && f_col % 4 == 0 && ((uintptr_t)proj & 15) == 0;
  dim3 grid(H, n_seqs, (dv + pb - 1) / pb);
#define FS(NR)                                                                                                     \
  cuca_launch(forget_scan_kernel<NR, false>, grid, dim3(threads), smem, stream, true, (const float*)proj, ld, q_col, \
              f_col, v_col, (const float*)nullptr, state, out, req_row0, req_count, slots, H, d, dv, ns, pb, tc, wide)
  if (nr == 4) FS(4);
  else if (nr == 8) FS(8);
  else if (nr == 16) FS(16);
  else FS(32);
#undef FS
  CUCA_CHECK_LAUNCH("forget_scan");
  return 0;
}

// Retention along every request's rows. proj: 32-bit rows of stride ld holding q heads at q_col, k heads at k_col (H
// heads of d each) and v heads at v_col (H heads of dv). The preparing kernel turns the first `rot` values of every q
// and k head by the row's position (pairs (i, i + rot/2); cos_t/sin_t: [table_rows, rot/2]) and multiplies k by
// k_scale, in place; the scan then runs S <- decay[h] S + k v^T, o = S^T q from the state in the request's slot
// (state: [slots, H, dv, d], out: [rows, H dv], both 32-bit).
CUCA_API int cuca_retention_scan(float* proj, int ld, int q_col, int k_col, int v_col, const float* decay,
                                 const float* cos_t, const float* sin_t, int table_rows, int rot, float k_scale,
                                 const int* positions, float* state, float* out, const int* seq_of_row,
                                 const int* req_row0, const int* req_count, const int* slots, int n_rows, int n_seqs,
                                 int H, int d, int dv, int* err, cudaStream_t stream) {
  if (n_seqs == 0 || n_rows == 0) return 0;
  CUCA_REQUIRE(H > 0 && d > 0 && dv > 0, "retention_scan: bad sizes heads=%d dim=%d vdim=%d", H, d, dv);
  CUCA_REQUIRE(rot >= 0 && rot <= d && rot % 2 == 0, "retention_scan: rotary size %d does not fit head size %d", rot, d);
  CUCA_REQUIRE(n_seqs <= 65535, "retention_scan: %d requests exceed the launch limit", n_seqs);
  int ns, nr;
  CUCA_REQUIRE(split_rows(d, (long long)n_seqs * H * dv, &ns, &nr), "retention_scan: %d key channels exceed %d", d, 32 * MAXR);
  {
    size_t blocks = ((size_t)n_rows * 2 * H * (d - rot / 2) + 255) / 256;
    blocks = blocks > 8192 ? 8192 : blocks;
    cuca_launch(retention_prepare_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, true, proj, ld, q_col, k_col,
                cos_t, sin_t, table_rows, rot, k_scale, positions, seq_of_row, n_rows, H, d, err);
    CUCA_CHECK_LAUNCH("retention_prepare");
  }
  int pb = block_threads(ns, nr) / ns;
  pb = pb > dv ? dv : pb;
  const int threads = (pb * ns + 31) / 32 * 32;
  const int per = (2 * ns * (nr == 4 ? 4 : nr + 4) + pb + 3) & ~3;
  int tc = 46000 / (2 * per * 4);
  tc = tc > 16 ? 16 : tc;
  CUCA_REQUIRE(tc >= 1, "retention_scan: a token of %d key channels does not fit shared memory", d);
  const size_t smem = (size_t)2 * tc * per * 4;
  const int wide = d % 4 == 0 && ld % 4 == 0 && q_col % 4 == 0 && k_col % 4 == 0 && ((uintptr_t)proj & 15) == 0;
  dim3 grid(H, n_seqs, (dv + pb - 1) / pb);
#define RS(NR)                                                                                                     \
  cuca_launch(forget_scan_kernel<NR, true>, grid, dim3(threads), smem, stream, true, (const float*)proj, ld, q_col,  \
              k_col, v_col, decay, state, out, req_row0, req_count, slots, H, d, dv, ns, pb, tc, wide)
  if (nr == 4) RS(4);
  else if (nr == 8) RS(8);
  else if (nr == 16) RS(16);
  else RS(32);
#undef RS
  CUCA_CHECK_LAUNCH("retention_scan");
  return 0;
}

// gate_act 0: the gate's factor is sigmoid(gate); 1: silu(gate). w null: no weight.
CUCA_API int cuca_head_norm_gate_act(const float* o, const float* w, int w_head, const void* gate, int gate_dtype,
                                     int ld_g, int gate_act, void* out, int out_dtype, int n_rows, int H, int dv,
                                     float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  const long long n_items = (long long)n_rows * H;
  dim3 grid((unsigned)((n_items + 7) / 8));
#define HNG(TG, TO)                                                                                                 \
  do {                                                                                                              \
    if (gate_act)                                                                                                   \
      cuca_launch(head_norm_gate_kernel<TG, TO, true>, grid, dim3(256), 0, stream, true, o, w, w_head,              \
                  (const TG*)gate, ld_g, (TO*)out, H, dv, eps, n_items);                                            \
    else                                                                                                            \
      cuca_launch(head_norm_gate_kernel<TG, TO, false>, grid, dim3(256), 0, stream, true, o, w, w_head,             \
                  (const TG*)gate, ld_g, (TO*)out, H, dv, eps, n_items);                                            \
  } while (0)
  if (gate_dtype == CUCA_F32 && out_dtype == CUCA_F32) HNG(float, float);
  else if (gate_dtype == CUCA_F32 && out_dtype == CUCA_BF16) HNG(float, __nv_bfloat16);
  else if (gate_dtype == CUCA_BF16 && out_dtype == CUCA_BF16) HNG(__nv_bfloat16, __nv_bfloat16);
  else CUCA_REQUIRE(false, "head_norm_gate: unsupported dtypes %d/%d", gate_dtype, out_dtype);
#undef HNG
  CUCA_CHECK_LAUNCH("head_norm_gate");
  return 0;
}

CUCA_API int cuca_head_norm_gate(const float* o, const float* w, int w_head, const void* gate, int gate_dtype, int ld_g,
                                 void* out, int out_dtype, int n_rows, int H, int dv, float eps, cudaStream_t stream) {
  return cuca_head_norm_gate_act(o, w, w_head, gate, gate_dtype, ld_g, 0, out, out_dtype, n_rows, H, dv, eps, stream);
}
