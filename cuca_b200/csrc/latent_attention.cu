// Attention over a cached low-rank latent: per token the cache holds one row [c | k_rot] (a normed latent of
// `rank` values and one rotated key part of `rot` values that every head shares) instead of keys and values per
// head. With k_h = U_h c and v_h = V_h c,
//   score = q_plain . (U_h c) + q_rot . k_rot = (U_h^T q_plain) . c + q_rot . k_rot,
//   out_h = V_h (sum_j p_j c_j),
// so a head's query is carried into the latent space once per row (`head_linear` with U_h^T), every head attends
// over the same cached rows, and the weighted sum of latents is taken out through V_h (`head_linear` again).
//   latent_prepare    norms c, rotates k_rot and the heads' q_rot (pairs (2i, 2i + 1) or (i, i + n/2)), writes the cache row
//   head_linear       out[t, h, :] = W_h a[t, h, :] for every head, optionally times sigmoid(gate)
//   latent_attention  plain form: one warp per (row, head), keys in tiles of 32 absolute positions
// Scores, softmax, norms and rotation are 32-bit; the cache has the compute dtype.
#include "common.cuh"
#include <math.h>

namespace {

// qkg: 32-bit rows of stride ld: [H x (dn + dr) queries | rank + dr down-projection | ...]. One block per row.
// qk: [rows, H, rank + dr] 32-bit; this kernel fills the last dr of every head with the rotated q_rot.
template <typename TC>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ qkg, int ld, int H, int dn, int dr, int rank,
                      const float* __restrict__ c_gain, float eps, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int table_rows, int rot_dims, int half_pairs,
                      float* __restrict__ qk,
                      TC* __restrict__ pool, int n_blocks, int bs, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_row, const int* __restrict__ tables, int table_stride, int* err) {
  __shared__ float red[8];
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int seq = seq_of_row[row];
  if (seq < 0) return;
  const int pos = positions[row];
  if (pos < 0 || pos >= table_rows) {
    if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_TOKEN_RANGE);
    return;
  }
  const int half = rot_dims >> 1;
  const float* cs = cos_t + (size_t)pos * half;
  const float* sn = sin_t + (size_t)pos * half;
  const float* qrow = qkg + (size_t)row * ld;
  const int Dk = rank + dr;
  // value j (< rot_dims) of a vector turned by the position: with its neighbour (2i, 2i + 1), or, half_pairs, with the
  // value half the rotated size away (i, i + rot_dims / 2)
  auto turned = [&](const float* src, int j) {
    if (half_pairs) {
      const bool up = j >= half;
      const int pr = up ? j - half : j;
      return up ? src[j] * cs[pr] + src[j - half] * sn[pr] : src[j] * cs[pr] - src[j + half] * sn[pr];
    }
    const int pr = j >> 1;
    return (j & 1) ? src[j] * cs[pr] + src[j - 1] * sn[pr] : src[j] * cs[pr] - src[j + 1] * sn[pr];
  };
  // the heads' rotated parts
  for (int i = threadIdx.x; i < H * dr; i += 256) {
    const int h = i / dr, j = i % dr;
    const float* src = qrow + (size_t)h * (dn + dr) + dn;
    qk[((size_t)row * H + h) * Dk + rank + j] = j < rot_dims ? turned(src, j) : src[j];
  }
  // the cache row
  const float* dkv = qrow + (size_t)H * (dn + dr);
  float s2 = 0.f;
  for (int i = threadIdx.x; i < rank; i += 256) s2 = fmaf(dkv[i], dkv[i], s2);
  s2 = warp_sum(s2);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s2;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)rank + eps);
  const int blk = tables[(size_t)seq * table_stride + pos / bs];
  if (blk < 0 || blk >= n_blocks) {
    if (threadIdx.x == 0 && err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
    return;
  }
  TC* dst = pool + ((size_t)blk * bs + (pos % bs)) * Dk;
  for (int i = threadIdx.x; i < rank; i += 256) dst[i] = from_f32<TC>(dkv[i] * inv * c_gain[i]);
  const float* kr = dkv + rank;
  for (int j = threadIdx.x; j < dr; j += 256) dst[rank + j] = from_f32<TC>(j < rot_dims ? turned(kr, j) : kr[j]);
}

// out[t, h, n] = sum_k a[t, h, k] w[h, n, k]  (* sigmoid(gate[t, h N + n])). Tiles of 64 rows x 64 outputs, 256
// threads with 4 x 4 results each, K in steps of 16 in ascending order whatever the tile a row falls in.
template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_linear_kernel(const float* __restrict__ a, int lda, int a_head, const TW* __restrict__ w, TO* __restrict__ out,
                   int ldo, int o_head, const float* __restrict__ gate, int ldg, int T, int N, int K) {
  __shared__ float As[16][64 + 4];
  __shared__ float Ws[16][64 + 4];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.z;
  const int t0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const TW* wh = w + (size_t)h * N * K;
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int e = threadIdx.x; e < 16 * 64; e += 256) {
      const int kk = e & 15, r = e >> 4;
      const int t = t0 + r, n = n0 + r, k = k0 + kk;
      As[kk][r] = (t < T && k < K) ? a[(size_t)t * lda + (size_t)h * a_head + k] : 0.f;
      Ws[kk][r] = (n < N && k < K) ? to_f32(wh[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (gate) v *= 1.f / (1.f + expf(-gate[(size_t)t * ldg + (size_t)h * N + n]));
      out[(size_t)t * ldo + (size_t)h * o_head + n] = from_f32<TO>(v);
    }
  }
}

// The same contraction on tensor cores (bfloat16 weights, many rows): tiles of 64 rows x 64 outputs, four warps of
// 16 rows each, K in steps of 32; `a` is rounded to bfloat16 on its way into shared memory, sums are 32-bit.
__device__ __forceinline__ void hl_ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void hl_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TO>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const float* __restrict__ a, int lda, int a_head, const __nv_bfloat16* __restrict__ w,
                       TO* __restrict__ out, int ldo, int o_head, const float* __restrict__ gate, int ldg, int T, int N,
                       int K) {
  constexpr int KS = 32, RSM = KS + 8;  // rows of 80 bytes: the eight rows of an ldmatrix fall into different banks
  __shared__ __align__(16) __nv_bfloat16 As[64 * RSM];
  __shared__ __align__(16) __nv_bfloat16 Ws[64 * RSM];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.z, t0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
  const int b_row = (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const __nv_bfloat16* wh = w + (size_t)h * N * K;
  const float* ah = a + (size_t)h * a_head;
  for (int k0 = 0; k0 < K; k0 += KS) {
    float av[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {  // 64 rows x 32 values, a row's 32 values side by side over a warp
      const int e = threadIdx.x + i * 128, r = e >> 5, kk = e & 31;
      av[i] = (t0 + r < T && k0 + kk < K) ? ah[(size_t)(t0 + r) * lda + k0 + kk] : 0.f;
    }
    __nv_bfloat16 wv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = threadIdx.x + i * 128, r = e >> 5, kk = e & 31;
      wv[i] = (n0 + r < N && k0 + kk < K) ? wh[(size_t)(n0 + r) * K + k0 + kk] : __float2bfloat16_rn(0.f);
    }
    __syncthreads();  // the step before is read to the end
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = threadIdx.x + i * 128, r = e >> 5, kk = e & 31;
      As[r * RSM + kk] = __float2bfloat16_rn(av[i]);
      Ws[r * RSM + kk] = wv[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KS; kk += 16) {
      uint32_t af[4];
      hl_ldsm_x4(af, As + (warp * 16 + a_row) * RSM + kk + a_col);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bf[4];
        hl_ldsm_x4(bf, Ws + (np * 16 + b_row) * RSM + kk + b_col);
        hl_mma(acc[2 * np], af, bf[0], bf[1]);
        hl_mma(acc[2 * np + 1], af, bf[2], bf[3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = t0 + warp * 16 + g + 8 * i;
    if (row >= T) continue;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int n = n0 + nt * 8 + 2 * t + j;
        if (n >= N) continue;
        float v = acc[nt][2 * i + j];
        if (gate) v *= 1.f / (1.f + expf(-gate[(size_t)row * ldg + (size_t)h * N + n]));
        out[(size_t)row * ldo + (size_t)h * o_head + n] = from_f32<TO>(v);
      }
  }
}

// The same contraction for up to 16 rows (single decoded tokens): a warp per (head, output) reads its weight row once
// and keeps a sum per row; the lanes split K. Used in the serving precision only: its sums run in another order
// than the tiled kernel's.
template <typename TW, typename TO>
__global__ void __launch_bounds__(128)
head_linear_rows_kernel(const float* __restrict__ a, int lda, int a_head, const TW* __restrict__ w,
                        TO* __restrict__ out, int ldo, int o_head, const float* __restrict__ gate, int ldg, int T,
                        int N, int K) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + (threadIdx.x >> 5), h = blockIdx.y;
  if (n >= N) return;
  float acc[16];
#pragma unroll
  for (int t = 0; t < 16; ++t) acc[t] = 0.f;
  const TW* wr = w + ((size_t)h * N + n) * K;
  const float* ah = a + (size_t)h * a_head;
  // four steps of K at once: their loads are in flight together (the kernel is all latency at these sizes)
#pragma unroll 4
  for (int k = lane; k < K; k += 32) {
    const float wv = to_f32(wr[k]);
#pragma unroll
    for (int t = 0; t < 16; ++t)
      if (t < T) acc[t] = fmaf(ah[(size_t)t * lda + k], wv, acc[t]);
  }
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    if (t < T) {
      float v = warp_sum(acc[t]);
      if (lane == 0) {
        if (gate) v *= 1.f / (1.f + expf(-gate[(size_t)t * ldg + (size_t)h * N + n]));
        out[(size_t)t * ldo + (size_t)h * o_head + n] = from_f32<TO>(v);
      }
    }
  }
}

// One warp per (row, head). qk: [rows, H, Dk] 32-bit; pool rows [Dk] per position; out: [rows, H, rank] 32-bit, the
// softmax-weighted sum of the first `rank` values of the visible cache rows. NACC * 32 >= rank.
template <typename TC, int NACC>
__global__ void __launch_bounds__(128)
latent_attention_kernel(const float* __restrict__ qk, float* __restrict__ out, const TC* __restrict__ pool,
                        int n_blocks, int bs, const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                        const int* __restrict__ tables, int table_stride, int H, int rank, int Dk, float scale,
                        int window, const float* __restrict__ sink, int* err) {
  extern __shared__ float qs[];  // [4][Dk]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y;
  const int head = blockIdx.x * 4 + warp;
  const int seq = seq_of_row[row];
  if (seq < 0 || head >= H) return;
  const int P = positions[row];
  float* qv = qs + warp * Dk;
  const float* qrow = qk + ((size_t)row * H + head) * Dk;
  for (int i = lane; i < Dk; i += 32) qv[i] = qrow[i];
  __syncwarp();
  int lo = 0;
  if (window > 0 && P - (window - 1) > 0) lo = P - (window - 1);
  float m = -INFINITY, l = 0.f;
  float acc[NACC];
#pragma unroll
  for (int c = 0; c < NACC; ++c) acc[c] = 0.f;
  const int* table = tables + (size_t)seq * table_stride;
  for (int t0 = (lo / 32) * 32; t0 <= P; t0 += 32) {
    const int kp = t0 + lane;
    bool valid = kp >= lo && kp <= P;
    long long base = -1;
    if (valid) {
      const int blk = table[kp / bs];
      if (blk < 0 || blk >= n_blocks) {
        if (err) atomicExch(err, CUCA_ERR_BLOCK_RANGE);
        valid = false;
      } else {
        base = ((long long)blk * bs + (kp % bs)) * Dk;
      }
    }
    float s = -INFINITY;
    if (valid) {
      const TC* kr = pool + base;
      float dot = 0.f;
      for (int i = 0; i < Dk; ++i) dot = fmaf(qv[i], to_f32(kr[i]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < NACC; ++c) acc[c] *= corr;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const long long bj = __shfl_sync(0xffffffffu, base, j);
      if (bj < 0) continue;
      const TC* vr = pool + bj;
#pragma unroll
      for (int c = 0; c < NACC; ++c) {
        const int dim = c * 32 + lane;
        if (dim < rank) acc[c] = fmaf(pj, to_f32(vr[dim]), acc[c]);
      }
    }
    m = m_new;
  }
  if (sink) {  // one more term exp(sink[head]) in the denominator, with no value
    const float m_new = fmaxf(m, sink[head]);
    const float corr = expf(m - m_new);
    l = l * corr + expf(sink[head] - m_new);
#pragma unroll
    for (int c = 0; c < NACC; ++c) acc[c] *= corr;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float* o = out + ((size_t)row * H + head) * rank;
#pragma unroll
  for (int c = 0; c < NACC; ++c) {
    const int dim = c * 32 + lane;
    if (dim < rank) o[dim] = acc[c] * inv;
  }
}

}  // namespace

CUCA_API int cuca_latent_max_rank() { return 1024; }

// half_pairs 0: rotated values pair as (2i, 2i + 1); 1: as (i, i + rot_dims / 2).
CUCA_API int cuca_latent_prepare_p(const float* qkg, int ld, int H, int dn, int dr, int rank, const float* c_gain,
                                   float eps, const float* cos_t, const float* sin_t, int table_rows, int rot_dims,
                                   int half_pairs, float* qk, void* pool, int pool_dtype, int n_blocks, int bs,
                                   const int* positions, const int* seq_of_row, const int* tables, int table_stride,
                                   int n_rows, int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(H > 0 && dn >= 0 && dr >= 0 && rank > 0, "latent_prepare: bad sizes");
  CUCA_REQUIRE(rot_dims % 2 == 0 && rot_dims <= dr, "latent_prepare: %d rotated dimensions do not fit %d", rot_dims, dr);
#define LP(TC)                                                                                                       \
  cuca_launch(latent_prepare_kernel<TC>, dim3(n_rows), dim3(256), 0, stream, true, qkg, ld, H, dn, dr, rank, c_gain, \
              eps, cos_t, sin_t, table_rows, rot_dims, half_pairs, qk, (TC*)pool, n_blocks, bs, positions, seq_of_row, \
              tables, table_stride, err)
  if (pool_dtype == CUCA_F32) LP(float);
  else if (pool_dtype == CUCA_BF16) LP(__nv_bfloat16);
  else CUCA_REQUIRE(false, "latent_prepare: unknown dtype %d", pool_dtype);
#undef LP
  CUCA_CHECK_LAUNCH("latent_prepare");
  return 0;
}

CUCA_API int cuca_latent_prepare(const float* qkg, int ld, int H, int dn, int dr, int rank, const float* c_gain,
                                 float eps, const float* cos_t, const float* sin_t, int table_rows, int rot_dims,
                                 float* qk, void* pool, int pool_dtype, int n_blocks, int bs, const int* positions,
                                 const int* seq_of_row, const int* tables, int table_stride, int n_rows, int* err,
                                 cudaStream_t stream) {
  return cuca_latent_prepare_p(qkg, ld, H, dn, dr, rank, c_gain, eps, cos_t, sin_t, table_rows, rot_dims, 0, qk, pool,
                               pool_dtype, n_blocks, bs, positions, seq_of_row, tables, table_stride, n_rows, err, stream);
}

// a: 32-bit, element (t, h, k) at a[t * lda + h * a_head + k]; w: [H, N, K]; out element (t, h, n) at
// out[t * ldo + h * o_head + n]; gate (or null): 32-bit, element (t, h, n) at gate[t * ldg + h * N + n].
CUCA_API int cuca_head_linear(const float* a, int lda, int a_head, const void* w, int w_dtype, void* out,
                              int out_dtype, int ldo, int o_head, const float* gate, int ldg, int T, int H, int N,
                              int K, cudaStream_t stream) {
  if (T == 0) return 0;
  CUCA_REQUIRE(H > 0 && N > 0 && K > 0 && H <= 65535, "head_linear: bad sizes heads=%d out=%d in=%d", H, N, K);
  if (T <= 16 && w_dtype == CUCA_BF16) {
    dim3 rows_grid((N + 3) / 4, H);
    if (out_dtype == CUCA_F32)
      cuca_launch(head_linear_rows_kernel<__nv_bfloat16, float>, rows_grid, dim3(128), 0, stream, true, a, lda, a_head,
                  (const __nv_bfloat16*)w, (float*)out, ldo, o_head, gate, ldg, T, N, K);
    else if (out_dtype == CUCA_BF16)
      cuca_launch(head_linear_rows_kernel<__nv_bfloat16, __nv_bfloat16>, rows_grid, dim3(128), 0, stream, true, a, lda,
                  a_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo, o_head, gate, ldg, T, N, K);
    else
      CUCA_REQUIRE(false, "head_linear: unsupported dtypes %d/%d", w_dtype, out_dtype);
    CUCA_CHECK_LAUNCH("head_linear");
    return 0;
  }
  dim3 grid((N + 63) / 64, (T + 63) / 64, H);
  CUCA_REQUIRE(grid.y <= 65535, "head_linear: %d rows exceed the launch limit", T);
  if (w_dtype == CUCA_BF16) {
    if (out_dtype == CUCA_F32)
      cuca_launch(head_linear_mma_kernel<float>, grid, dim3(128), 0, stream, true, a, lda, a_head,
                  (const __nv_bfloat16*)w, (float*)out, ldo, o_head, gate, ldg, T, N, K);
    else if (out_dtype == CUCA_BF16)
      cuca_launch(head_linear_mma_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, true, a, lda, a_head,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldo, o_head, gate, ldg, T, N, K);
    else
      CUCA_REQUIRE(false, "head_linear: unsupported dtypes %d/%d", w_dtype, out_dtype);
    CUCA_CHECK_LAUNCH("head_linear");
    return 0;
  }
#define HL(TW, TO)                                                                                               \
  cuca_launch(head_linear_kernel<TW, TO>, grid, dim3(256), 0, stream, true, a, lda, a_head, (const TW*)w, (TO*)out, \
              ldo, o_head, gate, ldg, T, N, K)
  if (w_dtype == CUCA_F32 && out_dtype == CUCA_F32) HL(float, float);
  else if (w_dtype == CUCA_BF16 && out_dtype == CUCA_F32) HL(__nv_bfloat16, float);
  else if (w_dtype == CUCA_BF16 && out_dtype == CUCA_BF16) HL(__nv_bfloat16, __nv_bfloat16);
  else CUCA_REQUIRE(false, "head_linear: unsupported dtypes %d/%d", w_dtype, out_dtype);
#undef HL
  CUCA_CHECK_LAUNCH("head_linear");
  return 0;
}

// sink (or null): 32-bit, one number per head: the softmax's denominator holds one more term exp(sink[head]) that has
// no value and is not scaled.
CUCA_API int cuca_latent_attention_s(const float* qk, float* out, const void* pool, int pool_dtype, int n_blocks, int bs,
                                     const int* positions, const int* seq_of_row, const int* tables, int table_stride,
                                     int n_rows, int H, int rank, int Dk, float scale, int window, const float* sink,
                                     int* err, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CUCA_REQUIRE(rank > 0 && rank <= Dk && rank <= cuca_latent_max_rank(), "latent_attention: latent size %d is outside 1..%d",
               rank, cuca_latent_max_rank());
  CUCA_REQUIRE(n_rows <= 65535, "latent_attention: %d rows in one step exceed the launch limit 65535", n_rows);
  dim3 grid((H + 3) / 4, n_rows);
  const size_t smem = (size_t)4 * Dk * sizeof(float);
#define LA(TC, NACC)                                                                                              \
  cuca_launch(latent_attention_kernel<TC, NACC>, grid, dim3(128), smem, stream, true, qk, out, (const TC*)pool,   \
              n_blocks, bs, positions, seq_of_row, tables, table_stride, H, rank, Dk, scale, window, sink, err)
#define LA_BY_RANK(TC)                    \
  do {                                    \
    if (rank <= 128) LA(TC, 4);           \
    else if (rank <= 256) LA(TC, 8);      \
    else if (rank <= 512) LA(TC, 16);     \
    else LA(TC, 32);                      \
  } while (0)
  if (pool_dtype == CUCA_F32) LA_BY_RANK(float);
  else if (pool_dtype == CUCA_BF16) LA_BY_RANK(__nv_bfloat16);
  else CUCA_REQUIRE(false, "latent_attention: unknown dtype %d", pool_dtype);
#undef LA_BY_RANK
#undef LA
  CUCA_CHECK_LAUNCH("latent_attention");
  return 0;
}

CUCA_API int cuca_latent_attention(const float* qk, float* out, const void* pool, int pool_dtype, int n_blocks, int bs,
                                   const int* positions, const int* seq_of_row, const int* tables, int table_stride,
                                   int n_rows, int H, int rank, int Dk, float scale, int window, int* err,
                                   cudaStream_t stream) {
  return cuca_latent_attention_s(qk, out, pool, pool_dtype, n_blocks, bs, positions, seq_of_row, tables, table_stride,
                                 n_rows, H, rank, Dk, scale, window, nullptr, err, stream);
}
