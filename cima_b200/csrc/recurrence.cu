// Linear recurrences over time with a matrix state per head, S [dim, vdim] in float32, carried from token to token
// and from step to step (state [slots, heads, dim, vdim], zeroed when a slot opens):
//
//   decay rule   S <- d_h S + k v^T;                       o = S^T q       d_h one constant a head; q, k, v through SiLU
//   delta rule   S <- diag(g_t) S;  u = beta_t (v - S^T k);  S <- S + k u^T;  o = S^T q
//                g_t one decay a key channel and token, beta_t one scalar a token; the read-out sees the token's write
//   gate rule    S <- diag(f_t) S + (1 - f_t) v^T;          o = S^T q       f_t = l + (1 - l) sigmoid(z_t + b) one forget gate
//                a key channel and token, made here from the projection z, a bias b and a lower bound l (both
//                [heads * dim]); what the gate forgets is what it lets in; q through SiLU, v as it is
//
// A block owns 32 neighbouring value channels (columns of S) of one (sequence, head); a column is shared by 8 lanes of a
// warp, each of which keeps an eighth of the column's rows in registers (rows 32 ii + 4 rg + e of row group rg, so that the
// lanes' 16-byte reads of k, q and g from shared memory cover 32 consecutive words).  The step's tokens are walked in
// order, 16 (8 for key sizes above 128) at a time: their k, q, g, v and beta are staged in shared memory, and the outputs
// leave through it in whole rows.  A sum over the key channels is a lane's own rows in ascending order in two interleaved
// partial sums, then a fixed shuffle tree over the 8 lanes, whatever the step: a token's result has the same bits whether
// its sequence came whole, in pieces or one token at a time, alone or in a batch.  Everything is float32 but the loads of
// q, k, v.
#include "common.cuh"

namespace {
constexpr int REC_SPLIT = 8;          // lanes that share a column
constexpr int REC_COLS = 32;          // columns of a block: 8 warps x 4
constexpr int REC_THREADS = 256;

__device__ __forceinline__ float rec_silu(float z) { return z / (1.0f + expf(-z)); }

__device__ __forceinline__ float rec_sum_over_lanes(float v) {        // over the 8 lanes of a column: lanes l, l ^ 4, l ^ 8, l ^ 16, ...
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

// CPT: columns a thread owns (its columns stand 32 apart).  With two, every read of k, q and g from shared memory serves
// both, but a block covers 64 columns and a sequence gets half as many blocks: measured slower for one prompt (1.2 ms
// against 0.97 ms a layer of 2,048 tokens at key and value size 128), so the launch takes one.
// MODE: 0 the decay rule, 1 the delta rule, 2 the gate rule.
template <typename TQ, typename TV, int DIMP, int MODE, int CPT>
__global__ void __launch_bounds__(REC_THREADS)
k_recurrence(const TQ* __restrict__ q, int ldq, const TQ* __restrict__ k, int ldk, const TV* __restrict__ v, int ldv,
             const float* __restrict__ g, const float* __restrict__ beta, const float* __restrict__ decay,
             float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
             float* __restrict__ out, int heads, int kv_heads, int dim, int vdim) {
  constexpr bool DELTA = MODE == 1, GATE = MODE == 2, CHANNEL = MODE != 0;      // CHANNEL: a decay a key channel and token
  cima_pdl_wait();
  constexpr int RP = DIMP / REC_SPLIT;                  // rows of a column that one lane keeps
  constexpr int CH = DIMP > 128 ? 8 : 16;               // tokens staged at a time
  constexpr int COLS = REC_COLS * CPT;                  // columns of the block
  __shared__ __align__(16) float sk[GATE ? 1 : CH][DIMP];     // the gate rule writes (1 - f) v: it needs no key
  __shared__ __align__(16) float sq[CH][DIMP];
  __shared__ __align__(16) float sg[CHANNEL ? CH : 1][DIMP];
  __shared__ float sv[CH][COLS];
  __shared__ float so[CH][COLS];
  __shared__ float sb[CH];
  const int seq = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * COLS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rg = lane >> 2, lc = warp * 4 + (lane & 3);  // row group; the thread's columns are col0 + lc + 32 x
  const int kvh = h / (heads / kv_heads);
  const int first = seq_first_row[seq], n = seq_first_row[seq + 1] - first;
  float* st = state + (((size_t)seq_slot[seq] * heads + h) * dim) * (size_t)vdim + col0 + lc;
  float S[CPT][RP];
#pragma unroll
  for (int x = 0; x < CPT; x++)
#pragma unroll
    for (int j = 0; j < RP; j++) {
      const int row = (j >> 2) * 32 + rg * 4 + (j & 3);
      S[x][j] = (col0 + lc + 32 * x < vdim && row < dim) ? st[(size_t)row * vdim + 32 * x] : 0.f;
    }
  const float dh = CHANNEL ? 1.f : decay[h];
  const int ldo = heads * vdim;

  // The next tokens' k, q, g, v and beta travel from global memory into registers while the current ones are worked on
  // from shared memory: every load of a stage is issued before any of them is waited for.
  constexpr int NLD = CH * DIMP / REC_THREADS;          // values of k (and of q, of g) a thread stages
  constexpr int NLV = (CH * COLS + REC_THREADS - 1) / REC_THREADS;
  // They wait there as they were loaded: a conversion in front of the work would wait for the load it converts.
  TQ rk[NLD], rq[NLD];
  TV rv[NLV];
  float rgt[DELTA ? NLD : 1], rb = 0.f;
  const TQ zero_q = cima_from_f32<TQ>(0.f);
  const TV zero_v = cima_from_f32<TV>(0.f);
  // The gate rule: k holds the gate's projection z, g its bias and decay its lower bound (the same for every token: a
  // thread stages the same channels in every round and keeps theirs).  A channel beyond the key size gets the bound 1: f = 1.
  float glow[GATE ? NLD : 1], gbias[GATE ? NLD : 1];
  if (GATE) {
#pragma unroll
    for (int r = 0; r < NLD; r++) {
      const int i = (threadIdx.x + r * REC_THREADS) % DIMP;
      glow[r] = i < dim ? decay[h * dim + i] : 1.f;
      gbias[r] = i < dim ? g[h * dim + i] : 0.f;
    }
  }
  auto fetch = [&](int t0) {
    const int nt = min(CH, n - t0);
#pragma unroll
    for (int r = 0; r < NLD; r++) {
      const int idx = threadIdx.x + r * REC_THREADS;
      const int tt = idx / DIMP, i = idx - tt * DIMP;
      const size_t row = (size_t)(first + t0 + tt);
      const bool ok = tt < nt && i < dim;
      rk[r] = ok ? k[row * ldk + (size_t)kvh * dim + i] : zero_q;
      rq[r] = ok ? q[row * ldq + (size_t)kvh * dim + i] : zero_q;
      if (DELTA) rgt[r] = ok ? g[(row * heads + h) * dim + i] : 1.f;
    }
#pragma unroll
    for (int r = 0; r < NLV; r++) {
      const int idx = threadIdx.x + r * REC_THREADS;
      const int tt = idx / COLS, cc = idx - tt * COLS;
      rv[r] = (tt < nt && col0 + cc < vdim) ? v[(size_t)(first + t0 + tt) * ldv + (size_t)h * vdim + col0 + cc] : zero_v;
    }
    if (DELTA) rb = (int)threadIdx.x < nt ? beta[(size_t)(first + t0 + threadIdx.x) * heads + h] : 0.f;
  };
  if (n > 0) fetch(0);

  for (int t0 = 0; t0 < n; t0 += CH) {
    const int nt = min(CH, n - t0);
    __syncthreads();
#pragma unroll
    for (int r = 0; r < NLD; r++) {
      const int idx = threadIdx.x + r * REC_THREADS;
      const int tt = idx / DIMP, i = idx - tt * DIMP;
      const float fk = cima_to_f32<TQ>(rk[r]), fq = cima_to_f32<TQ>(rq[r]);
      if (!GATE) sk[tt][i] = DELTA ? fk : rec_silu(fk);
      sq[tt][i] = DELTA ? fq : rec_silu(fq);
      if (DELTA) sg[tt][i] = rgt[r];
      if (GATE) sg[tt][i] = glow[r] + (1.0f - glow[r]) / (1.0f + expf(-(fk + gbias[r])));
    }
#pragma unroll
    for (int r = 0; r < NLV; r++) {
      const int idx = threadIdx.x + r * REC_THREADS;
      if (idx < CH * COLS) sv[idx / COLS][idx % COLS] = CHANNEL ? cima_to_f32<TV>(rv[r]) : rec_silu(cima_to_f32<TV>(rv[r]));
    }
    if (DELTA && threadIdx.x < CH) sb[threadIdx.x] = rb;
    __syncthreads();
    if (t0 + CH < n) fetch(t0 + CH);
    if constexpr (GATE) {
      // Nothing of a token's read-out feeds the next token's update, so four tokens are taken together: their updates
      // follow one another row by row (S <- u + f (S - u), which is f S + (1 - f) u), their sums over the lanes run side
      // by side.  A token's own arithmetic is the same wherever it stands among the four.
      static_assert(CPT == 1 || !GATE, "the gate rule runs one column a thread");
      constexpr int TB = 4;
      for (int tt = 0; tt < nt; tt += TB) {
        float o0[TB], o1[TB];
#pragma unroll
        for (int x = 0; x < TB; x++) {
          o0[x] = o1[x] = 0.f;
          if (tt + x < nt) {
            const float u = sv[tt + x][lc];
#pragma unroll
            for (int j = 0; j < RP; j += 4) {
              const int i = (j >> 2) * 32 + rg * 4;
              const float4 g4 = *reinterpret_cast<const float4*>(&sg[tt + x][i]);
              const float4 q4 = *reinterpret_cast<const float4*>(&sq[tt + x][i]);
              S[0][j] = fmaf(g4.x, S[0][j] - u, u); S[0][j + 1] = fmaf(g4.y, S[0][j + 1] - u, u);
              S[0][j + 2] = fmaf(g4.z, S[0][j + 2] - u, u); S[0][j + 3] = fmaf(g4.w, S[0][j + 3] - u, u);
              o0[x] = fmaf(S[0][j], q4.x, o0[x]); o1[x] = fmaf(S[0][j + 1], q4.y, o1[x]);
              o0[x] = fmaf(S[0][j + 2], q4.z, o0[x]); o1[x] = fmaf(S[0][j + 3], q4.w, o1[x]);
            }
          }
        }
#pragma unroll
        for (int x = 0; x < TB; x++) o0[x] += o1[x];
#pragma unroll
        for (int x = 0; x < TB; x++) o0[x] += __shfl_xor_sync(0xffffffffu, o0[x], 4);
#pragma unroll
        for (int x = 0; x < TB; x++) o0[x] += __shfl_xor_sync(0xffffffffu, o0[x], 8);
#pragma unroll
        for (int x = 0; x < TB; x++) o0[x] += __shfl_xor_sync(0xffffffffu, o0[x], 16);
        if (rg == 0) {
#pragma unroll
          for (int x = 0; x < TB; x++)
            if (tt + x < nt) so[tt + x][lc] = o0[x];
        }
      }
    } else {
#pragma unroll 2
    for (int tt = 0; tt < nt; tt++) {
      float u[CPT];
#pragma unroll
      for (int x = 0; x < CPT; x++) u[x] = sv[tt][lc + 32 * x];
      if (DELTA) {
        float p0[CPT], p1[CPT];
#pragma unroll
        for (int x = 0; x < CPT; x++) p0[x] = p1[x] = 0.f;
#pragma unroll
        for (int j = 0; j < RP; j += 4) {
          const int i = (j >> 2) * 32 + rg * 4;
          const float4 g4 = *reinterpret_cast<const float4*>(&sg[tt][i]);
          const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][i]);
#pragma unroll
          for (int x = 0; x < CPT; x++) {
            S[x][j] *= g4.x; S[x][j + 1] *= g4.y; S[x][j + 2] *= g4.z; S[x][j + 3] *= g4.w;
            p0[x] = fmaf(S[x][j], k4.x, p0[x]); p1[x] = fmaf(S[x][j + 1], k4.y, p1[x]);
            p0[x] = fmaf(S[x][j + 2], k4.z, p0[x]); p1[x] = fmaf(S[x][j + 3], k4.w, p1[x]);
          }
        }
        const float b = sb[tt];
#pragma unroll
        for (int x = 0; x < CPT; x++) u[x] = b * (u[x] - rec_sum_over_lanes(p0[x] + p1[x]));
      } else {
#pragma unroll
        for (int x = 0; x < CPT; x++)
#pragma unroll
          for (int j = 0; j < RP; j++) S[x][j] *= dh;
      }
      float o0[CPT], o1[CPT];
#pragma unroll
      for (int x = 0; x < CPT; x++) o0[x] = o1[x] = 0.f;
#pragma unroll
      for (int j = 0; j < RP; j += 4) {
        const int i = (j >> 2) * 32 + rg * 4;
        const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&sq[tt][i]);
#pragma unroll
        for (int x = 0; x < CPT; x++) {
          S[x][j] = fmaf(k4.x, u[x], S[x][j]); S[x][j + 1] = fmaf(k4.y, u[x], S[x][j + 1]);
          S[x][j + 2] = fmaf(k4.z, u[x], S[x][j + 2]); S[x][j + 3] = fmaf(k4.w, u[x], S[x][j + 3]);
          o0[x] = fmaf(S[x][j], q4.x, o0[x]); o1[x] = fmaf(S[x][j + 1], q4.y, o1[x]);
          o0[x] = fmaf(S[x][j + 2], q4.z, o0[x]); o1[x] = fmaf(S[x][j + 3], q4.w, o1[x]);
        }
      }
#pragma unroll
      for (int x = 0; x < CPT; x++) {
        const float o = rec_sum_over_lanes(o0[x] + o1[x]);
        if (rg == 0) so[tt][lc + 32 * x] = o;
      }
    }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * COLS; idx += REC_THREADS) {
      const int tt = idx / COLS, cc = idx - tt * COLS;
      if (col0 + cc < vdim) out[(size_t)(first + t0 + tt) * ldo + (size_t)h * vdim + col0 + cc] = so[tt][cc];
    }
  }
  cima_pdl_trigger();        // the tokens are done: the next kernel may be set up while the state is stored
#pragma unroll
  for (int x = 0; x < CPT; x++)
#pragma unroll
    for (int j = 0; j < RP; j++) {
      const int row = (j >> 2) * 32 + rg * 4 + (j & 3);
      if (col0 + lc + 32 * x < vdim && row < dim) st[(size_t)row * vdim + 32 * x] = S[x][j];
    }
}

template <typename TQ, typename TV, int MODE>
int launch_recurrence(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const float* g, const float* beta,
                      const float* decay, float* state, const int* seq_slot, const int* seq_first_row, float* out,
                      int n_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t stream) {
  const int cpt = 1;      // two columns a thread (CPT 2) measured slower: half as many blocks, and the chain of a token is no shorter
  const dim3 grid((vdim + REC_COLS * cpt - 1) / (REC_COLS * cpt), heads, n_seqs);
#define RUN_C(D, C) return cima_launch(k_recurrence<TQ, TV, D, MODE, C>, grid, dim3(REC_THREADS), (size_t)0, stream, 1, (const TQ*)q, ldq, (const TQ*)k, ldk, \
                                       (const TV*)v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, heads, kv_heads, dim, vdim)
#define RUN(D) { RUN_C(D, 1); }
  if (dim <= 32) RUN(32);
  if (dim <= 64) RUN(64);
  if (dim <= 128) RUN(128);
  RUN(256);
#undef RUN
#undef RUN_C
}

// Everything of the delta rule that is computed per token before the recurrence, in float32:
//   qn = q / sqrt(sum q^2 + 1e-6) * dim^(-1/2),  kn = k / sqrt(sum k^2 + 1e-6)            per head of q and k
//   g  = exp(-exp(A_log[h]) * softplus(a + dt_bias)),  beta = sigmoid(b)
// A warp takes one unit of a row: a head of q, a head of k, or a head's decays with its beta; a block four units.  (One
// block a row, its warps walking the row's units one after another, took 17 us for the 8 rows of a decode step: a chain of
// some dozen trips to memory on 8 SMs.)
template <typename TA>
__global__ void __launch_bounds__(128)
k_delta_prepare(const TA* __restrict__ qk, int ldqk, const TA* __restrict__ a, int lda, const TA* __restrict__ b, int ldb,
                const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ qn, float* __restrict__ kn,
                float* __restrict__ g, float* __restrict__ beta, int heads, int kv_heads, int dim) {
  cima_pdl_wait();
  cima_pdl_trigger();        // the next kernel may be set up while this one runs (it waits for this one's end itself)
  const size_t row = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int u = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (u < 2 * kv_heads) {                                       // a head of q (u < kv_heads) or of k
    const TA* src = qk + row * ldqk + (size_t)u * dim;
    float x[8];                                                 // dim <= 256: eight values a lane
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = lane + 32 * j;
      x[j] = i < dim ? cima_to_f32<TA>(src[i]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) ss = fmaf(x[j], x[j], ss);
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = (1.0f / sqrtf(ss + 1e-6f)) * (u < kv_heads ? 1.0f / sqrtf((float)dim) : 1.0f);
    float* dst = u < kv_heads ? qn + (row * kv_heads + u) * dim : kn + (row * kv_heads + (u - kv_heads)) * dim;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = lane + 32 * j;
      if (i < dim) dst[i] = x[j] * r;
    }
  } else if (u < 2 * kv_heads + heads) {                        // a head's decays and its beta
    const int h = u - 2 * kv_heads;
    const float rate = expf(A_log[h]);
    float z[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = lane + 32 * j;
      z[j] = i < dim ? cima_to_f32<TA>(a[row * lda + (size_t)h * dim + i]) + dt_bias[h * dim + i] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = lane + 32 * j;
      if (i < dim) {
        const float sp = z[j] > 20.f ? z[j] : log1pf(expf(z[j]));
        g[(row * heads + h) * dim + i] = expf(-rate * sp);
      }
    }
    if (lane == 0) beta[row * heads + h] = 1.0f / (1.0f + expf(-cima_to_f32<TA>(b[row * ldb + h])));
  }
}
}  // namespace

// delta != 0: q, k float32 [T, kv_heads * dim] (prepared), v (vdtype) [T, ldv], g [T, heads * dim], beta [T, heads].
// delta == 0: q, k, v of one dtype (vdtype), SiLU applied here; decay [heads].  out [T, heads * vdim] float32.
// delta == 2 (the gate rule): q and k of v's dtype, k holding the gate's projection; g its bias and decay its lower bound,
// both [heads * dim] and shared by all tokens.
extern "C" int cima_recurrence(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, int vdtype,
                               const float* g, const float* beta, const float* decay, float* state, const int* seq_slot,
                               const int* seq_first_row, float* out, int T, int n_seqs, int heads, int kv_heads, int dim,
                               int vdim, int delta, cudaStream_t stream) {
  if (T <= 0 || n_seqs <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads > 65535 || n_seqs > 65535)
    return cima_fail(CIMA_E_SIZE, "recurrence: %d heads on %d key heads in %d sequences are not accepted", heads, kv_heads, n_seqs);
  if (dim <= 0 || dim > 256 || vdim <= 0) return cima_fail(CIMA_E_SIZE, "recurrence: key size %d must lie in 1..256 and value size %d be positive", dim, vdim);
  if (!state || !out || !q || !k || !v) return cima_fail(CIMA_E_ARG, "recurrence: q, k, v, the state and the output are needed");
  if (delta == 2) {
    if (!g || !decay) return cima_fail(CIMA_E_ARG, "recurrence: the gate rule needs the gate's bias and lower bound");
    int rc2;
    if (vdtype == CIMA_F32) rc2 = launch_recurrence<float, float, 2>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else if (vdtype == CIMA_BF16) rc2 = launch_recurrence<__nv_bfloat16, __nv_bfloat16, 2>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else return cima_fail(CIMA_E_DTYPE, "recurrence: dtype code %d is neither float32 nor bfloat16", vdtype);
    return rc2 ? rc2 : cima_launch_result();
  }
  if (delta && (!g || !beta)) return cima_fail(CIMA_E_ARG, "recurrence: the delta rule needs the tokens' decays and step sizes");
  if (!delta && !decay) return cima_fail(CIMA_E_ARG, "recurrence: the decay rule needs the heads' decays");
  int rc;
  if (delta) {
    if (vdtype == CIMA_F32) rc = launch_recurrence<float, float, 1>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else if (vdtype == CIMA_BF16) rc = launch_recurrence<float, __nv_bfloat16, 1>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else return cima_fail(CIMA_E_DTYPE, "recurrence: dtype code %d is neither float32 nor bfloat16", vdtype);
  } else {
    if (vdtype == CIMA_F32) rc = launch_recurrence<float, float, 0>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else if (vdtype == CIMA_BF16) rc = launch_recurrence<__nv_bfloat16, __nv_bfloat16, 0>(q, ldq, k, ldk, v, ldv, g, beta, decay, state, seq_slot, seq_first_row, out, n_seqs, heads, kv_heads, dim, vdim, stream);
    else return cima_fail(CIMA_E_DTYPE, "recurrence: dtype code %d is neither float32 nor bfloat16", vdtype);
  }
  return rc ? rc : cima_launch_result();
}

// qk [T, ldqk]: q's heads then k's (2 * kv_heads * dim values of a row); a [T, lda]: heads * dim; b [T, ldb]: heads.
extern "C" int cima_delta_prepare(const void* qk, int ldqk, const void* a, int lda, const void* b, int ldb, int dtype,
                                  const float* A_log, const float* dt_bias, float* qn, float* kn, float* g, float* beta,
                                  int T, int heads, int kv_heads, int dim, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || dim <= 0 || dim > 256) return cima_fail(CIMA_E_SIZE, "delta_prepare: heads %d and key heads %d must be positive, the key size %d in 1..256", heads, kv_heads, dim);
  if (T > 65535) return cima_fail(CIMA_E_SIZE, "delta_prepare: %d rows exceed one launch; the caller cuts them", T);
  const dim3 grid((unsigned)((2 * kv_heads + heads + 3) / 4), (unsigned)T);
  int rc;
  if (dtype == CIMA_F32) rc = cima_launch(k_delta_prepare<float>, grid, dim3(128), (size_t)0, stream, 1, (const float*)qk, ldqk, (const float*)a, lda, (const float*)b, ldb, A_log, dt_bias, qn, kn, g, beta, heads, kv_heads, dim);
  else if (dtype == CIMA_BF16) rc = cima_launch(k_delta_prepare<__nv_bfloat16>, grid, dim3(128), (size_t)0, stream, 1, (const __nv_bfloat16*)qk, ldqk, (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)b, ldb, A_log, dt_bias, qn, kn, g, beta, heads, kv_heads, dim);
  else return cima_fail(CIMA_E_DTYPE, "delta_prepare: dtype code %d is neither float32 nor bfloat16", dtype);
  return rc ? rc : cima_launch_result();
}
