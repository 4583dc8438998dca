// What an attention over latents needs beside the attention itself.
//
// latent_append: a row's compressed vector r (R values, a slice of a projection's output) becomes the latent
//   c = r / sqrt(mean(r^2) + eps) * g        (float32; one rounding at the store)
// and is written to the sequence's page at the row's position.  The pages hold ONE vector per position
// ([pages, 1, 1, page_size, R]): keys and values are both projected from it, so it is stored once.
//
// head_linear: the same small matrix product for every head,
//   out[t, h, n] = sum_k a[t, h, k] * w[h, n, k]        a: [T, heads, K] in rows of lda; out: [T, heads, N] in rows of ldo
// (a head of a row may be wider than K or N: `ha` and `ho` values lie between one head's start and the next in a and out)
// which moves a query into the latents' space (w = the key projection's head, transposed) and an attention
// result out of it (w = the value projection's head).  FFMA with one float32 accumulator per output in ascending
// k: the same bits for a row whatever comes with it.  It serves the 32-bit path at every size and the
// bfloat16 path for the few rows of a decode step; many bfloat16 rows are the caller's to give to the library's
// batched product, as it does with the other products of many rows.
#include "common.cuh"

// ------------------------------------------------------------------------------------------- latent_append
template <typename TA>
__global__ void __launch_bounds__(128)
k_latent_append(const TA* __restrict__ raw, int ld, const float* __restrict__ g, float eps, TA* __restrict__ cache,
                CimaPaged pg, const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                const int* __restrict__ seq_slot, int R) {
  cima_pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const TA* r = raw + (size_t)row * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = cima_to_f32<TA>(r[i]); ss += v * v; }
  const float total = cima_block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)R + eps);
  TA* dst = cache + pg.offset(seq_slot[row_seq[row]], row_pos[row], 0, 0);
  for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = cima_from_f32<TA>(cima_to_f32<TA>(r[i]) * inv * g[i]);
}

// raw: [T, ld] of `dtype`, the R values of a row starting at `raw`; cache: the layer's pages [pages, 1, 1, page_size, R].
extern "C" int cima_latent_append(const void* raw, int dtype, int ld, const float* g, float eps, void* cache,
                                  const int* table, int table_width, int ring, int page_size, const int* row_pos,
                                  const int* row_seq, const int* seq_slot, int T, int R, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (R <= 0 || ld < R) return cima_fail(CIMA_E_SIZE, "latent_append: %d values in rows of %d", R, ld);
  if (!cache || !table) return cima_fail(CIMA_E_ARG, "latent_append: the layer's pages and their block table are needed");
  CimaPaged pg{table, table_width, ring, page_size, 1, R, 1};
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_latent_append<float>, dim3(T), dim3(128), (size_t)0, stream, 1, (const float*)raw, ld, g, eps, (float*)cache, pg, row_pos, row_seq, seq_slot, R);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_latent_append<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, stream, 1, (const __nv_bfloat16*)raw, ld, g, eps, (__nv_bfloat16*)cache, pg, row_pos, row_seq, seq_slot, R);
  else return cima_fail(CIMA_E_DTYPE, "latent_append: dtype code %d is neither float32 nor bfloat16", dtype);
  if (rc) return rc;
  return cima_launch_result();
}

// ------------------------------------------------------------------------------------------- head_linear
template <typename TA>
__global__ void __launch_bounds__(256)
k_head_linear(const TA* __restrict__ A, const TA* __restrict__ W, TA* __restrict__ out, int M, int N, int K, int lda, int ldo,
              int ha, int ho) {
  cima_pdl_wait();
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int head = blockIdx.z;
  A += (size_t)head * ha;
  W += (size_t)head * N * K;
  out += (size_t)head * ho;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int r = 0; r < 4; r++) {
      const int idx = threadIdx.x + r * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float a = 0.f, w = 0.f;
      if (k < K) {
        if (m0 + row < M) a = cima_to_f32<TA>(A[(size_t)(m0 + row) * lda + k]);
        if (n0 + row < N) w = cima_to_f32<TA>(W[(size_t)(n0 + row) * K + k]);
      }
      As[kk][row] = a;
      Ws[kk][row] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * ldo + n] = cima_from_f32<TA>(acc[i][j]);
    }
  }
}

// Few rows (a decode step): a block takes 32 outputs n of one head; warp m of the block computes them for row m
// of A, lane l the output n0 + l: the lane walks its row of the head's matrix once (16-byte loads, a chunk of 64 k in
// registers at a time) against the row of A in shared memory (every lane reads the same value: a broadcast), one
// float32 accumulator in ascending k.  All warps of a block read the same weight rows, which the first one brings
// into the first-level cache.  The work is a few hundred KB of weights; its time is latency, so the chain of a
// thread is kept short (K fused multiply-adds) and the blocks many.
constexpr int HL_FEW_ROWS = 8;
constexpr int HL_FEW_K = 64;          // k of a row that a thread holds in registers at a time

template <typename TA> struct HlVec;
template <> struct HlVec<float> { static constexpr int N = 4; };
template <> struct HlVec<__nv_bfloat16> { static constexpr int N = 8; };

// A decode step's latents can be appended by the same launch (both read the projection that ran just before): one
// more row of blocks, of which the first does what k_latent_append does, warp m for row m.
template <typename TA>
struct LatentJob {
  const TA* raw;                // null: no job
  int ld;
  const float* g;
  float eps;
  TA* cache;
  CimaPaged pg;
  const int *row_pos, *row_seq, *seq_slot;
  int R;
};

template <typename TA>
__global__ void __launch_bounds__(32 * HL_FEW_ROWS)
k_head_linear_few(const TA* __restrict__ A, const TA* __restrict__ W, TA* __restrict__ out, int M, int N, int K, int lda, int ldo,
                  int ha, int ho, int vec, LatentJob<TA> job) {
  extern __shared__ __align__(16) float a_sh[];         // [M][Kp], Kp = K rounded up to 4
  const int Kp = (K + 3) & ~3;
  const int head = blockIdx.y;
  const int lane = threadIdx.x & 31, m = threadIdx.x >> 5;
  if (job.raw && blockIdx.y == gridDim.y - 1) {
    if (blockIdx.x != 0) return;
    cima_pdl_wait();
    const TA* r = job.raw + (size_t)m * job.ld;
    float ss = 0.f;
    for (int i = lane; i < job.R; i += 32) { const float v = cima_to_f32<TA>(r[i]); ss += v * v; }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)job.R + job.eps);
    TA* dst = job.cache + job.pg.offset(job.seq_slot[job.row_seq[m]], job.row_pos[m], 0, 0);
    for (int i = lane; i < job.R; i += 32) dst[i] = cima_from_f32<TA>(cima_to_f32<TA>(r[i]) * inv * job.g[i]);
    return;
  }
  const int n = blockIdx.x * 32 + lane;
  const bool live = n < N;
  const TA* wr = W + ((size_t)head * N + (live ? n : 0)) * K;
  constexpr int V = HlVec<TA>::N;
  float w[HL_FEW_K];
  // the first chunk of the weights does not depend on the kernel before this one: it is requested before the wait
  const int kn0 = min(HL_FEW_K, K);
  if (vec && kn0 == HL_FEW_K) {
#pragma unroll
    for (int q = 0; q < HL_FEW_K / V; q++) {
      const uint4 raw = *reinterpret_cast<const uint4*>(wr + q * V);
      const TA* e = reinterpret_cast<const TA*>(&raw);
#pragma unroll
      for (int i = 0; i < V; i++) w[q * V + i] = cima_to_f32<TA>(e[i]);
    }
  } else {
#pragma unroll
    for (int q = 0; q < HL_FEW_K; q++) w[q] = q < kn0 ? cima_to_f32<TA>(wr[q]) : 0.f;
  }
  cima_pdl_wait();
  A += (size_t)head * ha;
  for (int e = threadIdx.x; e < M * Kp; e += blockDim.x) {
    const int r = e / Kp, k = e - r * Kp;
    a_sh[e] = k < K ? cima_to_f32<TA>(A[(size_t)r * lda + k]) : 0.f;
  }
  __syncthreads();
  const float* ar = a_sh + m * Kp;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += HL_FEW_K) {
    const int kn = min(HL_FEW_K, K - k0);
    if (k0 > 0) {
      if (vec && kn == HL_FEW_K) {
#pragma unroll
        for (int q = 0; q < HL_FEW_K / V; q++) {
          const uint4 raw = *reinterpret_cast<const uint4*>(wr + k0 + q * V);
          const TA* e = reinterpret_cast<const TA*>(&raw);
#pragma unroll
          for (int i = 0; i < V; i++) w[q * V + i] = cima_to_f32<TA>(e[i]);
        }
      } else {
#pragma unroll
        for (int q = 0; q < HL_FEW_K; q++) w[q] = q < kn ? cima_to_f32<TA>(wr[k0 + q]) : 0.f;
      }
    }
    // (chunks beyond the row's end were loaded as zeros, and A's row is padded with zeros to a multiple of 4)
#pragma unroll
    for (int q = 0; q < HL_FEW_K; q += 4) {
      if (q < kn) {
        const float4 a = *reinterpret_cast<const float4*>(ar + k0 + q);
        acc = fmaf(a.x, w[q], acc);
        acc = fmaf(a.y, w[q + 1], acc);
        acc = fmaf(a.z, w[q + 2], acc);
        acc = fmaf(a.w, w[q + 3], acc);
      }
    }
  }
  if (live) out[(size_t)m * ldo + (size_t)head * ho + n] = cima_from_f32<TA>(acc);
}

// a [M, heads, K] in rows of lda, w [heads, N, K] contiguous, out [M, heads, N] in rows of ldo; all of `dtype`.
// raw (may be null) ... R: the arguments of cima_latent_append for the same M rows, done by the same launch; only for
// the few rows of a decode step (M <= 8).
static int head_linear_impl(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                            int ldo, int ha, int ho, const void* raw, int ld_raw, const float* g, float eps, void* cache, const int* table,
                            int table_width, int ring, int page_size, const int* row_pos, const int* row_seq,
                            const int* seq_slot, int R, cudaStream_t stream);

extern "C" int cima_head_linear(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                                int ldo, int ha, int ho, cudaStream_t stream) {
  return head_linear_impl(a, w, out, dtype, M, heads, N, K, lda, ldo, ha, ho, nullptr, 0, nullptr, 0.f, nullptr, nullptr, 0, 0, 0,
                          nullptr, nullptr, nullptr, 0, stream);
}

extern "C" int cima_head_linear_append(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                                       int ldo, const void* raw, int ld_raw, const float* g, float eps, void* cache,
                                       const int* table, int table_width, int ring, int page_size, const int* row_pos,
                                       const int* row_seq, const int* seq_slot, int R, cudaStream_t stream) {
  if (M > HL_FEW_ROWS || (size_t)M * (K + 3) * 4 > 48 * 1024)
    return cima_fail(CIMA_E_SIZE, "head_linear_append: %d rows of %d values; the launch that also appends takes at most %d rows", M, K, HL_FEW_ROWS);
  if (!raw || !g || !cache || !table || R <= 0 || ld_raw < R)
    return cima_fail(CIMA_E_ARG, "head_linear_append: the compressed rows (%d values in rows of %d), the norm's weight, the pages and their table are needed", R, ld_raw);
  return head_linear_impl(a, w, out, dtype, M, heads, N, K, lda, ldo, K, N, raw, ld_raw, g, eps, cache, table, table_width, ring,
                          page_size, row_pos, row_seq, seq_slot, R, stream);
}

static int head_linear_impl(const void* a, const void* w, void* out, int dtype, int M, int heads, int N, int K, int lda,
                            int ldo, int ha, int ho, const void* raw, int ld_raw, const float* g, float eps, void* cache, const int* table,
                            int table_width, int ring, int page_size, const int* row_pos, const int* row_seq,
                            const int* seq_slot, int R, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (heads <= 0 || N <= 0 || K <= 0) return cima_fail(CIMA_E_SIZE, "head_linear: %d heads, N %d and K %d must be positive", heads, N, K);
  if (ha < K || ho < N || lda < (heads - 1) * ha + K || ldo < (heads - 1) * ho + N)
    return cima_fail(CIMA_E_SIZE, "head_linear: rows of (%d, %d) do not hold %d heads of (%d, %d) at every (%d, %d) values", lda, ldo, heads, K, N, ha, ho);
  if (heads > 65535 || (M + 63) / 64 > 65535) return cima_fail(CIMA_E_SIZE, "head_linear: %d heads / %d rows exceed one launch", heads, M);
  int rc;
  if (M <= HL_FEW_ROWS && (size_t)M * (K + 3) * 4 <= 48 * 1024) {
    const dim3 grid((N + 31) / 32, heads + (raw ? 1 : 0));
    const CimaPaged pg{table, table_width, ring, page_size, 1, R, 1};
    const size_t smem = (size_t)M * ((K + 3) & ~3) * sizeof(float);
    const int esz = dtype == CIMA_F32 ? 4 : 2;
    const int vec = (((uintptr_t)w & 15) == 0 && ((size_t)K * esz) % 16 == 0) ? 1 : 0;      // every row of w starts on 16 bytes
    if (dtype == CIMA_F32) rc = cima_launch(k_head_linear_few<float>, grid, dim3(32 * M), smem, stream, 1, (const float*)a, (const float*)w, (float*)out, M, N, K, lda, ldo, ha, ho, vec,
                                                LatentJob<float>{(const float*)raw, ld_raw, g, eps, (float*)cache, pg, row_pos, row_seq, seq_slot, R});
    else if (dtype == CIMA_BF16) rc = cima_launch(k_head_linear_few<__nv_bfloat16>, grid, dim3(32 * M), smem, stream, 1, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, lda, ldo, ha, ho, vec,
                                                  LatentJob<__nv_bfloat16>{(const __nv_bfloat16*)raw, ld_raw, g, eps, (__nv_bfloat16*)cache, pg, row_pos, row_seq, seq_slot, R});
    else return cima_fail(CIMA_E_DTYPE, "head_linear: dtype code %d is neither float32 nor bfloat16", dtype);
  } else if (dtype == CIMA_BF16) {
    const dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    rc = cima_launch(k_head_linear<__nv_bfloat16>, grid, dim3(256), (size_t)0, stream, 1, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, lda, ldo, ha, ho);
  } else if (dtype == CIMA_F32) {
    const dim3 grid((N + 63) / 64, (M + 63) / 64, heads);
    rc = cima_launch(k_head_linear<float>, grid, dim3(256), (size_t)0, stream, 1, (const float*)a, (const float*)w, (float*)out, M, N, K, lda, ldo, ha, ho);
  } else return cima_fail(CIMA_E_DTYPE, "head_linear: dtype code %d is neither float32 nor bfloat16", dtype);
  if (rc) return rc;
  return cima_launch_result();
}

// ------------------------------------------------------------------------------------------- latent_prepare, rope_rows
// latent_prepare: a row of a latent attention's first product is [first | R | rot]: with cq, the first part is a query
// latent, cq = rms(part) * q_norm; c = rms(second part) * c_norm; the third part is rotated at the row's position.
// [c | rotated part] goes to the row's place in the one-plane pages (heads of R + rot values) and, with `step`, twice
// into a row of the step's own buffer (as key and as value of a prompt's attention).  A block a row: warp 0 norms the
// query latent, warp 1 the latent, warp 2 rotates; sums of squares by a shuffle tree, float32 throughout, one rounding
// at each store.  Pairs: (2i, 2i + 1) where `interleaved`, else (i, i + rot / 2); sine and cosine times `amp`.
template <typename TA>
__global__ void __launch_bounds__(96)
k_latent_prepare(const TA* __restrict__ ql, int ld, int first, const float* __restrict__ q_norm, TA* __restrict__ cq, int q_rank,
                 const float* __restrict__ c_norm, float eps, int R, int rot, const float* __restrict__ inv_freq, float amp,
                 int interleaved, TA* __restrict__ cache_in, CimaPaged pg, const int* __restrict__ row_pos,
                 const int* __restrict__ row_seq, const int* __restrict__ seq_slot, const int* __restrict__ seq_len,
                 TA* __restrict__ step, int step_ld, int step_col) {
  cima_pdl_wait();
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const TA* r = ql + (size_t)row * ld;
  const int pos = row_pos[row];
  TA* cache = cache_in;
  // in a ring of pages a position whose place a later position of the same step takes is not written at all
  if (cache && pg.ring && pos + pg.ring * pg.page_size < seq_len[row_seq[row]]) cache = nullptr;
  TA* dst = cache ? cache + pg.offset(seq_slot[row_seq[row]], pos, 0, 0) : nullptr;
  TA* s1 = step ? step + (size_t)row * step_ld + step_col : nullptr;
  TA* s2 = s1 ? s1 + R + rot : nullptr;
  if (warp == 0) {
    if (!cq) return;
    float ss = 0.f;
    for (int i = lane; i < q_rank; i += 32) { const float v = cima_to_f32<TA>(r[i]); ss = fmaf(v, v, ss); }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
    TA* out = cq + (size_t)row * q_rank;
    for (int i = lane; i < q_rank; i += 32) out[i] = cima_from_f32<TA>(cima_to_f32<TA>(r[i]) * inv * q_norm[i]);
  } else if (warp == 1) {
    const TA* c = r + first;
    float ss = 0.f;
    for (int i = lane; i < R; i += 32) { const float v = cima_to_f32<TA>(c[i]); ss = fmaf(v, v, ss); }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    for (int i = lane; i < R; i += 32) {
      const TA v = cima_from_f32<TA>(cima_to_f32<TA>(c[i]) * inv * c_norm[i]);
      if (dst) dst[i] = v;
      if (s1) { s1[i] = v; s2[i] = v; }
    }
  } else {
    const TA* k = r + first + R;
    const int half = rot >> 1;
    for (int i = lane; i < half; i += 32) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      sn *= amp; cs *= amp;
      const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
      const float a = cima_to_f32<TA>(k[ia]), b = cima_to_f32<TA>(k[ib]);
      const TA ra = cima_from_f32<TA>(a * cs - b * sn), rb = cima_from_f32<TA>(b * cs + a * sn);
      if (dst) { dst[R + ia] = ra; dst[R + ib] = rb; }
      if (s1) { s1[R + ia] = ra; s1[R + ib] = rb; s2[R + ia] = ra; s2[R + ib] = rb; }
    }
  }
}

extern "C" int cima_latent_prepare(const void* ql, int dtype, int ld, int first, const float* q_norm, void* cq, int q_rank,
                                   const float* c_norm, float eps, int R, int rot, const float* inv_freq, float amp, int interleaved,
                                   void* cache, const int* table, int table_width, int ring, int page_size, const int* row_pos,
                                   const int* row_seq, const int* seq_slot, const int* seq_len, void* step, int step_ld, int step_col,
                                   int T, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (R <= 0 || rot < 0 || (rot & 1) || first < 0 || ld < first + R + rot)
    return cima_fail(CIMA_E_SIZE, "latent_prepare: rows of %d values do not hold %d + %d + an even %d", ld, first, R, rot);
  if (cq && (q_rank <= 0 || q_rank > first || !q_norm)) return cima_fail(CIMA_E_ARG, "latent_prepare: a query latent of %d values within the first %d, with its norm's weight, is needed", q_rank, first);
  if (!c_norm || (rot && !inv_freq)) return cima_fail(CIMA_E_ARG, "latent_prepare: the latent norm's weight and the rotation's frequencies are needed");
  if (!cache || !table || !seq_len) return cima_fail(CIMA_E_ARG, "latent_prepare: the layer's pages, their block table and the sequences' lengths are needed");
  if (step && step_ld < step_col + 2 * (R + rot)) return cima_fail(CIMA_E_SIZE, "latent_prepare: the step's rows of %d values do not hold two copies from column %d on", step_ld, step_col);
  CimaPaged pg{table, table_width, ring, page_size, 1, R + rot, 1};
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_latent_prepare<float>, dim3(T), dim3(96), (size_t)0, stream, 1, (const float*)ql, ld, first, q_norm, (float*)cq, q_rank, c_norm, eps, R, rot, inv_freq, amp, interleaved, (float*)cache, pg, row_pos, row_seq, seq_slot, seq_len, (float*)step, step_ld, step_col);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_latent_prepare<__nv_bfloat16>, dim3(T), dim3(96), (size_t)0, stream, 1, (const __nv_bfloat16*)ql, ld, first, q_norm, (__nv_bfloat16*)cq, q_rank, c_norm, eps, R, rot, inv_freq, amp, interleaved, (__nv_bfloat16*)cache, pg, row_pos, row_seq, seq_slot, seq_len, (__nv_bfloat16*)step, step_ld, step_col);
  else return cima_fail(CIMA_E_DTYPE, "latent_prepare: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}

// rope_rows: out[t, h * o_head + o_off + j] = the j-th of `rot` values q[t, h * q_head + q_off + ...] rotated at row t's position.
template <typename TA>
__global__ void __launch_bounds__(128)
k_rope_rows(const TA* __restrict__ q, int ldq, int q_off, int q_head, TA* __restrict__ out, int ldo, int o_off, int o_head, int heads,
            int rot, const float* __restrict__ inv_freq, float amp, int interleaved, const int* __restrict__ row_pos) {
  cima_pdl_wait();
  const int row = blockIdx.x;
  const int half = rot >> 1;
  const float pos = (float)row_pos[row];
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    sn *= amp; cs *= amp;
    const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
    const TA* src = q + (size_t)row * ldq + (size_t)h * q_head + q_off;
    TA* dst = out + (size_t)row * ldo + (size_t)h * o_head + o_off;
    const float a = cima_to_f32<TA>(src[ia]), b = cima_to_f32<TA>(src[ib]);
    dst[ia] = cima_from_f32<TA>(a * cs - b * sn);
    dst[ib] = cima_from_f32<TA>(b * cs + a * sn);
  }
}

extern "C" int cima_rope_rows(const void* q, int dtype, int ldq, int q_off, int q_head, void* out, int ldo, int o_off, int o_head,
                              int heads, int rot, const float* inv_freq, float amp, int interleaved, const int* row_pos, int T,
                              cudaStream_t stream) {
  if (T <= 0 || rot == 0) return 0;
  if (heads <= 0 || rot < 0 || (rot & 1) || q_off < 0 || o_off < 0 || ldq < (heads - 1) * q_head + q_off + rot || ldo < (heads - 1) * o_head + o_off + rot)
    return cima_fail(CIMA_E_SIZE, "rope_rows: %d heads of %d rotating values do not fit rows of (%d, %d)", heads, rot, ldq, ldo);
  if (!inv_freq || !row_pos) return cima_fail(CIMA_E_ARG, "rope_rows: the frequencies and the rows' positions are needed");
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_rope_rows<float>, dim3(T), dim3(128), (size_t)0, stream, 1, (const float*)q, ldq, q_off, q_head, (float*)out, ldo, o_off, o_head, heads, rot, inv_freq, amp, interleaved, row_pos);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_rope_rows<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, stream, 1, (const __nv_bfloat16*)q, ldq, q_off, q_head, (__nv_bfloat16*)out, ldo, o_off, o_head, heads, rot, inv_freq, amp, interleaved, row_pos);
  else return cima_fail(CIMA_E_DTYPE, "rope_rows: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}
