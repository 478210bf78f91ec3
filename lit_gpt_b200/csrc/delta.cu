// Gated delta rule: a recurrent layer whose state is one dk x dv matrix S per head, kept in fp32.
//
//   per token:  S <- g * S          (g: one decay per head, or one per head and key channel acting on the rows of S)
//               u  = beta * (v - S^T k)
//               S <- S + k u^T
//               o  = S^T q          (the read-out sees the token's own write)
//   with beta = sigmoid(b) and g = exp(-exp(A_log) * softplus(a + dt_bias)) computed here in fp32 from the raw projections.
//
// The columns of S never mix: column j evolves from (k, q, g, beta) and v[j] alone.  So the work of one (sequence, head) is
// split over columns -- a group of LPC lanes owns one column, each lane holding dk / LPC of its numbers in registers -- and
// over CTAs (column blocks); the host picks LPC (see b200_delta_rule).  Time is walked in order: tiles of tokens are staged in shared memory (keys, queries, decays
// already turned into g) while the previous tile is walked; per token every lane group does three short dot products that
// share one reduction (o = (g S)^T q + (k . q) u needs no second pass over the updated state) and one update.  One kernel serves
// prompts (many rows per sequence) and decoding (one row: the cost is reading and writing S once).
//
// A sequence that starts at position 0 starts from S = 0 whatever its slot holds.  The state is stored in the order the
// kernel's lane groups read whole 32-byte sectors: element (key i, column j) of a head at ((i / L) * dv + j) * L + i % L with
// L = 4, 8, 16 or 32 by key size (b200_delta_rule_state_floats).
//
// b200_gated_rms_heads is the step after the read-out: per head, o / sqrt(mean(o^2) + eps) * weight * gate(z) with
// gate = silu or sigmoid.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kDrThreads = 128, kDrTile = 1024;   // floats of keys (queries, decays) staged per tile

__host__ __device__ inline int delta_lpc(int dk) { return dk <= 64 ? 4 : dk <= 128 ? 8 : dk <= 256 ? 16 : 32; }
__host__ __device__ inline int delta_key_rows(int dk) { const int l = delta_lpc(dk); return (dk + l - 1) / l; }

struct DrArgs {
  const float* q; const float* k; const float* v;
  int64_t ldq, ldk, ldv;
  const void* beta_in; int64_t ld_beta;
  const void* decay_in; int64_t ld_decay;
  const void* a_log; const void* dt_bias;
  float* state; int64_t state_slot_stride;
  float* out; int64_t ldo;
  const int4* seqs;
  int heads, kv_heads, dk, dv;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// LPC lanes share one column of S, each holding KPL of its numbers (key i = r * LPC + lane); L is the group size of the stored
// layout, which does not depend on how the kernel spreads a column over lanes.
template <typename T, int LPC, int KPL, bool CHANNEL>
__global__ void __launch_bounds__(kDrThreads) delta_rule_kernel(DrArgs A, int L) {
  constexpr int kDrKPL = KPL;
  constexpr int DKP = KPL * LPC;               // padded key size
  constexpr int TT = kDrTile / DKP;            // tokens per staged tile
  constexpr int COLS = kDrThreads / LPC;       // columns per CTA
  constexpr int NIT = TT * DKP / kDrThreads;   // key elements of a tile per thread (8)
  constexpr int NV = (TT * COLS + kDrThreads - 1) / kDrThreads;   // value elements of a tile per thread
  extern __shared__ __align__(16) float dr_smem[];
  float* const ks = dr_smem;                   // [TT][DKP]
  float* const qs = ks + TT * DKP;             // [TT][DKP]
  float* const gs = qs + TT * DKP;             // [TT][DKP] (channel decay) or [TT]
  float* const vs = gs + (CHANNEL ? TT * DKP : TT);   // [TT][COLS]
  float* const bs = vs + TT * COLS;            // [TT]
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x, sub = tid % LPC, cl = tid / LPC;
  const int h = blockIdx.y, hk = h / (A.heads / A.kv_heads);
  const int4 sq = A.seqs[blockIdx.z];
  const int first = sq.x, len = sq.y, pos0 = sq.z, slot = sq.w;
  const int col = (int)blockIdx.x * COLS + cl;
  const bool col_ok = col < A.dv;
  const int dk = A.dk, dv = A.dv;
  const int krows = (dk + L - 1) / L;           // rows of L keys in the stored layout
  float* const st = A.state + (int64_t)slot * A.state_slot_stride + (int64_t)h * krows * L * dv;
  auto where = [&](int r) -> int64_t {          // key r * LPC + sub of this lane's column; -1 past the padded key size
    const int i = r * LPC + sub;
    return i < krows * L ? ((int64_t)(i / L) * dv + col) * L + i % L : -1;
  };

  float S[kDrKPL];
#pragma unroll
  for (int r = 0; r < kDrKPL; ++r) {
    const int64_t w = where(r);
    S[r] = (pos0 > 0 && col_ok && w >= 0) ? st[w] : 0.f;
  }

  const float neg_a = -expf(load_as_float(reinterpret_cast<const T*>(A.a_log), h));
  const T* const bias = reinterpret_cast<const T*>(A.dt_bias);
  const T* const dec = reinterpret_cast<const T*>(A.decay_in);
  const T* const bet = reinterpret_cast<const T*>(A.beta_in);

  // A tile's inputs travel global -> registers -> shared memory: the loads of tile n + 1 are issued before the tokens of tile n
  // are walked, so their latency hides behind the recurrence; the decays are turned into g on the way into shared memory.
  float rk[NIT], rq[NIT], rd[CHANNEL ? NIT : 1], rbias[CHANNEL ? NIT : 1], rv[NV], rb = 0.f, rg = 0.f;
  if (CHANNEL) {
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int i = (tid + it * kDrThreads) % DKP;
      rbias[it] = i < dk ? load_as_float(bias, (int64_t)h * dk + i) : 0.f;
    }
  }
  const float hbias = CHANNEL ? 0.f : load_as_float(bias, h);
  auto load_tile = [&](int t0) {
    const int nt = min(TT, len - t0);
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int idx = tid + it * kDrThreads, t = idx / DKP, i = idx - t * DKP;
      const bool ok = t < nt && i < dk;
      const int64_t row = first + t0 + t;
      rk[it] = ok ? A.k[row * A.ldk + (int64_t)hk * dk + i] : 0.f;
      rq[it] = ok ? A.q[row * A.ldq + (int64_t)hk * dk + i] : 0.f;
      if (CHANNEL) rd[it] = ok ? load_as_float(dec, row * A.ld_decay + (int64_t)h * dk + i) : 0.f;
    }
#pragma unroll
    for (int iv = 0; iv < NV; ++iv) {
      const int idx = tid + iv * kDrThreads, t = idx / COLS, c = (int)blockIdx.x * COLS + (idx - t * COLS);
      rv[iv] = (idx < TT * COLS && t < nt && c < dv) ? A.v[(int64_t)(first + t0 + t) * A.ldv + (int64_t)h * dv + c] : 0.f;
    }
    if (tid < TT) {
      const bool ok = tid < nt;
      const int64_t row = first + t0 + tid;
      rb = ok ? load_as_float(bet, row * A.ld_beta + h) : -INFINITY;
      if (!CHANNEL) rg = ok ? load_as_float(dec, row * A.ld_decay + h) : 0.f;
    }
  };
  auto store_tile = [&]() {
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int idx = tid + it * kDrThreads;
      ks[idx] = rk[it];
      qs[idx] = rq[it];
      if (CHANNEL) gs[idx] = expf(neg_a * softplus_f(rd[it] + rbias[it]));
    }
#pragma unroll
    for (int iv = 0; iv < NV; ++iv) {
      const int idx = tid + iv * kDrThreads;
      if (idx < TT * COLS) vs[idx] = rv[iv];
    }
    if (tid < TT) {
      bs[tid] = 1.0f / (1.0f + expf(-rb));
      if (!CHANNEL) gs[tid] = expf(neg_a * softplus_f(rg + hbias));
    }
  };

  load_tile(0);
  for (int t0 = 0; t0 < len; t0 += TT) {
    const int nt = min(TT, len - t0);
    __syncthreads();                       // the previous tile's tokens are done with shared memory
    store_tile();
    __syncthreads();
    if (t0 + TT < len) load_tile(t0 + TT);
    for (int t = 0; t < nt; ++t) {
      const float* kt = ks + t * DKP + sub;
      const float* qt = qs + t * DKP + sub;
      // with D = g S (decayed state):  u = beta (v - D^T k),  S = D + k u^T,  o = S^T q = D^T q + (k . q) u
      // so the three dot products over the key axis are independent and share the rounds of one reduction; with few numbers per
      // lane each is summed in two interleaved halves (measured: 0.66 -> 0.57 us per token there, a loss with 16 per lane)
      constexpr int NA = KPL <= 8 ? 2 : 1;
      float kr[kDrKPL];
      float dk_[2] = {0.f, 0.f}, dq_[2] = {0.f, 0.f}, kq_[2] = {0.f, 0.f};
      if (CHANNEL) {
        const float* gt = gs + t * DKP + sub;
#pragma unroll
        for (int r = 0; r < kDrKPL; ++r) {
          kr[r] = kt[r * LPC];
          const float qv = qt[r * LPC];
          S[r] *= gt[r * LPC];
          dk_[r % NA] = fmaf(S[r], kr[r], dk_[r % NA]);
          dq_[r % NA] = fmaf(S[r], qv, dq_[r % NA]);
          kq_[r % NA] = fmaf(kr[r], qv, kq_[r % NA]);
        }
      } else {
        const float g = gs[t];
#pragma unroll
        for (int r = 0; r < kDrKPL; ++r) {
          kr[r] = kt[r * LPC];
          const float qv = qt[r * LPC];
          S[r] *= g;
          dk_[r % NA] = fmaf(S[r], kr[r], dk_[r % NA]);
          dq_[r % NA] = fmaf(S[r], qv, dq_[r % NA]);
          kq_[r % NA] = fmaf(kr[r], qv, kq_[r % NA]);
        }
      }
      float dks = dk_[0] + dk_[1], dqs = dq_[0] + dq_[1], kqs = kq_[0] + kq_[1];
#pragma unroll
      for (int o = LPC / 2; o > 0; o >>= 1) {
        dks += __shfl_xor_sync(0xffffffffu, dks, o);
        dqs += __shfl_xor_sync(0xffffffffu, dqs, o);
        kqs += __shfl_xor_sync(0xffffffffu, kqs, o);
      }
      const float u = bs[t] * (vs[t * COLS + cl] - dks);
#pragma unroll
      for (int r = 0; r < kDrKPL; ++r) S[r] = fmaf(kr[r], u, S[r]);
      if (sub == 0 && col_ok) A.out[(int64_t)(first + t0 + t) * A.ldo + (int64_t)h * dv + col] = fmaf(kqs, u, dqs);
    }
  }
  if (col_ok) {
#pragma unroll
    for (int r = 0; r < kDrKPL; ++r) {
      const int64_t w = where(r);
      if (w >= 0) st[w] = S[r];
    }
  }
}

template <typename T, int LPC, int KPL>
cudaError_t delta_launch(const DrArgs& A, bool channel, int n_seqs, cudaStream_t st) {
  constexpr int DKP = KPL * LPC, TT = kDrTile / DKP, COLS = kDrThreads / LPC;
  const dim3 grid((unsigned)((A.dv + COLS - 1) / COLS), (unsigned)A.heads, (unsigned)n_seqs);
  const int L = delta_lpc(A.dk);
  if (channel) {
    const size_t smem = (size_t)(3 * TT * DKP + TT * COLS + TT) * sizeof(float);
    return launch(delta_rule_kernel<T, LPC, KPL, true>, grid, dim3(kDrThreads), smem, st, A, L);
  }
  const size_t smem = (size_t)(2 * TT * DKP + TT + TT * COLS + TT) * sizeof(float);
  return launch(delta_rule_kernel<T, LPC, KPL, false>, grid, dim3(kDrThreads), smem, st, A, L);
}

// out[row, h, :] = T( o / sqrt(mean(o^2) + eps) * weight * gate(z[row, h, :]) ); one warp per (row, head)
template <typename T>
__global__ void __launch_bounds__(128) gated_rms_heads_kernel(const float* __restrict__ o, int64_t ldo, const T* __restrict__ z, int64_t ldz,
                                                              const T* __restrict__ weight, T* __restrict__ out, int64_t ld_out, int heads,
                                                              int dv, int gate, float eps) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int h = (int)blockIdx.y * 4 + (threadIdx.x >> 5);
  if (h >= heads) return;
  const int64_t row = blockIdx.x;
  const float* orow = o + row * ldo + (int64_t)h * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(orow[i], orow[i], ss);
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int i = lane; i < dv; i += 32) {
    const float zz = load_as_float(z, row * ldz + (int64_t)h * dv + i);
    const float sg = 1.0f / (1.0f + expf(-zz));
    store_from_float(out, row * ld_out + (int64_t)h * dv + i, orow[i] * rstd * load_as_float(weight, i) * (gate == 1 ? zz * sg : sg));
  }
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int64_t b200_delta_rule_state_floats(int dk, int dv) { return (int64_t)delta_key_rows(dk) * delta_lpc(dk) * dv; }

int b200_delta_rule(const b200_delta_rule_args* a, b200_stream_t stream) {
  B200_CHECK_ARG(a && a->q && a->k && a->v && a->beta_in && a->decay_in && a->a_log && a->dt_bias && a->state && a->out && a->seqs,
                 "b200_delta_rule: null pointer");
  B200_CHECK_ARG(a->n_seqs > 0 && a->n_seqs <= 65535 && a->heads > 0 && a->heads <= 65535 && a->kv_heads > 0 && a->heads % a->kv_heads == 0,
                 "b200_delta_rule: bad head counts");
  B200_CHECK_ARG(a->dk > 0 && a->dk <= 512 && a->dv > 0, "b200_delta_rule: key size must be 1 .. 512");
  B200_CHECK_ARG((reinterpret_cast<uintptr_t>(a->seqs) & 15) == 0, "b200_delta_rule: seqs must be 16-byte aligned");
  const DrArgs A{a->q, a->k, a->v, a->ldq, a->ldk, a->ldv, a->beta_in, a->ld_beta, a->decay_in, a->ld_decay, a->a_log, a->dt_bias,
                 a->state, a->state_slot_stride, a->out, a->ldo, reinterpret_cast<const int4*>(a->seqs), a->heads, a->kv_heads, a->dk, a->dv};
  const bool ch = a->channel_decay != 0;
  cudaStream_t st = (cudaStream_t)stream;
  // Two ways to spread a column over lanes.  Few lanes with 16 numbers each: three reduction rounds per token and whole
  // 128-byte lines of state per warp -- best for single tokens and for the per-head decay.  A prompt with per-channel decays
  // carries a third staged array and the softplus / exponential of every decay: there a column on 16 or 32 lanes with 4 or 8
  // numbers each (four times the warps) measured faster (0.66 against 0.85 us per token at 8 heads of 128 x 128).
  // (that is with 64 to 128 CTAs of the narrow split; once those alone fill the GPU, more warps only add reduction rounds)
  const int64_t narrow_ctas = (int64_t)((a->dv + kDrThreads / delta_lpc(a->dk) - 1) / (kDrThreads / delta_lpc(a->dk))) * a->heads * a->n_seqs;
  const bool wide = ch && a->max_rows > 1 && a->dk > 32 && a->dk <= 256 && narrow_ctas < (int64_t)sm_count() * 3 / 2;
  B200_FLOAT_TYPES(a->dtype, T, {
    if (wide) {
      if (a->dk <= 64) B200_CUDA((delta_launch<T, 16, 4>(A, ch, a->n_seqs, st)));
      else if (a->dk <= 128) B200_CUDA((delta_launch<T, 32, 4>(A, ch, a->n_seqs, st)));
      else B200_CUDA((delta_launch<T, 32, 8>(A, ch, a->n_seqs, st)));
    } else {
      const int lpc = delta_lpc(a->dk);
      if (lpc == 4) B200_CUDA((delta_launch<T, 4, 16>(A, ch, a->n_seqs, st)));
      else if (lpc == 8) B200_CUDA((delta_launch<T, 8, 16>(A, ch, a->n_seqs, st)));
      else if (lpc == 16) B200_CUDA((delta_launch<T, 16, 16>(A, ch, a->n_seqs, st)));
      else B200_CUDA((delta_launch<T, 32, 16>(A, ch, a->n_seqs, st)));
    }
  });
  return B200_OK;
}

int b200_gated_rms_heads(const float* o, int64_t ldo, const void* z, int64_t ldz, const void* weight, void* out, int64_t ld_out, int64_t rows,
                         int heads, int dv, int gate, float eps, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(o && z && weight && out, "b200_gated_rms_heads: null pointer");
  B200_CHECK_ARG(rows > 0 && rows <= 0x7fffffff && heads > 0 && (heads + 3) / 4 <= 65535 && dv > 0, "b200_gated_rms_heads: bad shape");
  B200_CHECK_ARG(gate == 1 || gate == 2, "b200_gated_rms_heads: gate is 1 (silu) or 2 (sigmoid)");
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(gated_rms_heads_kernel<T>, dim3((unsigned)rows, (unsigned)((heads + 3) / 4)), dim3(128), 0,
                                               (cudaStream_t)stream, o, ldo, (const T*)z, ldz, (const T*)weight, (T*)out, ld_out, heads, dv, gate, eps)));
  return B200_OK;
}

}  // extern "C"
