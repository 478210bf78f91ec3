// Short causal convolution over time on the channels of a projection, with the per-head step that follows it fused in.
//
//   y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c]            (zeros before a sequence's first position)
//
// A step brings the rows of several sequences packed into one matrix (seqs[s] = {first row, rows, first position, state
// slot}).  Inputs from before the step's first row come from the sequence's tail: the last taps - 1 projected rows that
// earlier steps left in its state slot.  Whether a tap lies before the sequence start, in the tail or in the step is decided
// by its POSITION alone, so a slot that another sequence used before needs no clearing.
//
// The channels form up to three groups of heads (e.g. queries, keys, values); one warp owns one (row, head) and applies
// after the convolution, in fp32:
//   act  : none | silu
//   post : none
//        | rotate + norm : rotary positions on the first rot_dims dimensions, interleaved pairs (2i, 2i + 1) turned by the
//                          angle position * inv_freq[i], cos and sin times rot_mscale; then x / sqrt(mean(x^2) + eps)
//        | unit          : x / sqrt(sum(x^2) + eps)
//   and a final multiplier post_scale.
// b200_conv_tail_update then stores each sequence's new tail.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kCvThreads = 128, kCvMaxTaps = 8, kCvMaxGroups = 3, kCvMaxIt = 8;   // head size <= 64 * kCvMaxIt

struct CvGroup {
  const void* w;
  void* out;
  int64_t ld_out;
  const double* inv_freq;
  int col0, heads, dim, act, post, rot_dims, out_f32;
  float rot_mscale, post_scale, eps;
};

struct CvParams {
  CvGroup g[kCvMaxGroups];
  int n_groups, taps, total_heads;
};

// two neighbouring elements at once when the caller vouches for the alignment (one 4- or 8-byte access)
template <typename T>
__device__ __forceinline__ void load_pair(const T* p, int64_t i, bool pair, bool second, float& a, float& b);
template <>
__device__ __forceinline__ void load_pair<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i, bool pair, bool second, float& a, float& b) {
  if (pair) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(p + i);
    a = bf16lo(v);
    b = bf16hi(v);
  } else {
    a = __bfloat162float(p[i]);
    b = second ? __bfloat162float(p[i + 1]) : 0.f;
  }
}
template <>
__device__ __forceinline__ void load_pair<float>(const float* p, int64_t i, bool pair, bool second, float& a, float& b) {
  if (pair) {
    const float2 v = *reinterpret_cast<const float2*>(p + i);
    a = v.x;
    b = v.y;
  } else {
    a = p[i];
    b = second ? p[i + 1] : 0.f;
  }
}

// NIT: 64-element pieces of the widest head; TAPS: the number of taps when it is one of the unrolled ones, else 0 (read at run time)
template <typename T, int NIT, int TAPS>
__global__ void __launch_bounds__(kCvThreads) short_conv_kernel(const T* __restrict__ in, int64_t ld_in, CvParams P,
                                                                 const T* __restrict__ tail, int64_t tail_slot_stride, int tail_cols,
                                                                 const int4* __restrict__ seqs, const int* __restrict__ row_seq, int pairs) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  int hh = (int)blockIdx.y * (kCvThreads / 32) + (threadIdx.x >> 5);
  if (hh >= P.total_heads) return;
  int gi = 0;
  while (gi + 1 < P.n_groups && hh >= P.g[gi].heads) { hh -= P.g[gi].heads; ++gi; }
  const CvGroup& G = P.g[gi];
  const int64_t row = blockIdx.x;
  const int4 sq = seqs[row_seq[row]];
  const int r = (int)(row - sq.x);            // row within the step's part of its sequence
  const int pos = sq.z + r;
  const int taps = TAPS ? TAPS : P.taps;
  const T* tl = tail + (int64_t)sq.w * tail_slot_stride;
  const T* wt = reinterpret_cast<const T*>(G.w);
  const int c_head = G.col0 + hh * G.dim;     // first channel of this head among the convolved columns
  const bool pair = (pairs & 1) != 0;
  const bool wvec = TAPS == 4 && (pairs & 2) != 0;   // the eight taps of two neighbouring channels in one 16-byte (fp32: 32-byte) access

  float val[NIT][2];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    const int d = it * 64 + lane * 2;
    float acc0 = 0.f, acc1 = 0.f;
    if (d < G.dim) {
      const bool second = d + 1 < G.dim;
      const int c = c_head + d;
      const T* wc = wt + (int64_t)(hh * G.dim + d) * taps;
      float wf[8];
      if (wvec) load8(wc, wf);
#pragma unroll
      for (int j = 0; j < (TAPS ? TAPS : kCvMaxTaps + 1); ++j) {
        if (!TAPS && j >= taps) break;
        const int back = taps - 1 - j;       // how many positions before this row
        float u0 = 0.f, u1 = 0.f;
        if (back <= pos) {                   // else: before the sequence's first token, zero
          if (back <= r) load_pair(in, (row - back) * ld_in + c, pair, second, u0, u1);
          else load_pair(tl, (int64_t)(taps - 1 - (back - r)) * tail_cols + c, pair, second, u0, u1);   // tail row taps-1-k: the k-th row before the step
        }
        if (wvec) {
          acc0 = fmaf(wf[j & 3], u0, acc0);
          acc1 = fmaf(wf[4 + (j & 3)], u1, acc1);
        } else {
          acc0 = fmaf(load_as_float(wc, j), u0, acc0);
          if (second) acc1 = fmaf(load_as_float(wc, taps + j), u1, acc1);
        }
      }
      if (G.act == 1) {
        acc0 = acc0 / (1.0f + expf(-acc0));
        acc1 = acc1 / (1.0f + expf(-acc1));
      }
    }
    val[it][0] = acc0;
    val[it][1] = acc1;
  }
  if (G.post == 1) {
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int d = it * 64 + lane * 2;
      if (d + 1 < G.rot_dims && d + 1 < G.dim) {
        // the angle in double, reduced to [-pi, pi] before the fp32 sine and cosine: exact to fp32 at any position
        double a = (double)pos * G.inv_freq[d >> 1];
        a -= 6.283185307179586476925286766559 * rint(a * 0.15915494309189533576888376337251);
        float sn, cs;
        sincosf((float)a, &sn, &cs);
        sn *= G.rot_mscale;
        cs *= G.rot_mscale;
        const float u = val[it][0], v = val[it][1];
        val[it][0] = u * cs - v * sn;
        val[it][1] = v * cs + u * sn;
      }
    }
  }
  if (G.post != 0) {
#pragma unroll
    for (int it = 0; it < NIT; ++it) ss += val[it][0] * val[it][0] + val[it][1] * val[it][1];   // lanes past dim hold zeros
    ss = warp_sum(ss);
  }
  float mul = G.post_scale;
  if (G.post == 1) mul *= 1.0f / sqrtf(ss / (float)G.dim + G.eps);
  else if (G.post == 2) mul *= 1.0f / sqrtf(ss + G.eps);
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int d = it * 64 + lane * 2 + e;
      if (d < G.dim) {
        const int64_t o = row * G.ld_out + (int64_t)hh * G.dim + d;
        if (G.out_f32) reinterpret_cast<float*>(G.out)[o] = val[it][e] * mul;
        else store_from_float(reinterpret_cast<T*>(G.out), o, val[it][e] * mul);
      }
    }
  }
}

template <typename T, int NIT>
cudaError_t short_conv_launch(int taps, dim3 grid, cudaStream_t st, const T* in, int64_t ld_in, const CvParams& P, const T* tail,
                              int64_t tail_slot_stride, int tail_cols, const int4* seqs, const int* row_seq, int pairs) {
  switch (taps) {
    case 2: return launch(short_conv_kernel<T, NIT, 2>, grid, dim3(kCvThreads), 0, st, in, ld_in, P, tail, tail_slot_stride, tail_cols, seqs, row_seq, pairs);
    case 3: return launch(short_conv_kernel<T, NIT, 3>, grid, dim3(kCvThreads), 0, st, in, ld_in, P, tail, tail_slot_stride, tail_cols, seqs, row_seq, pairs);
    case 4: return launch(short_conv_kernel<T, NIT, 4>, grid, dim3(kCvThreads), 0, st, in, ld_in, P, tail, tail_slot_stride, tail_cols, seqs, row_seq, pairs);
    default: return launch(short_conv_kernel<T, NIT, 0>, grid, dim3(kCvThreads), 0, st, in, ld_in, P, tail, tail_slot_stride, tail_cols, seqs, row_seq, pairs);
  }
}

// tail[slot][i] <- the (taps - 1 - i)-th last projected row of the sequence after this step, i = 0 .. taps - 2; rows that
// the step did not bring move up from the old tail.  One thread per (sequence, channel) reads all it needs before writing.
template <typename T>
__global__ void __launch_bounds__(256) conv_tail_kernel(const T* __restrict__ in, int64_t ld_in, T* __restrict__ tail,
                                                        int64_t tail_slot_stride, int tail_cols, int taps, const int4* __restrict__ seqs) {
  griddep_launch();
  griddep_wait();
  const int c = (int)blockIdx.x * 256 + threadIdx.x;
  if (c >= tail_cols) return;
  const int4 sq = seqs[blockIdx.y];
  const int L = sq.y, n = taps - 1;
  T* tl = tail + (int64_t)sq.w * tail_slot_stride;
  T keep[kCvMaxTaps];
#pragma unroll
  for (int i = 0; i < kCvMaxTaps; ++i) {
    if (i >= n) break;
    const int back = n - 1 - i;                 // rows before the sequence's last row
    if (back < L) keep[i] = in[(int64_t)(sq.x + L - 1 - back) * ld_in + c];
    else if (i + L < n) keep[i] = tl[(int64_t)(i + L) * tail_cols + c];
    else keep[i] = tl[(int64_t)i * tail_cols + c];   // unreachable: back >= L implies i + L < n
  }
#pragma unroll
  for (int i = 0; i < kCvMaxTaps; ++i) {
    if (i >= n) break;
    tl[(int64_t)i * tail_cols + c] = keep[i];
  }
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

int b200_short_conv(const void* in, int64_t ld_in, const b200_conv_group* groups, int n_groups, int taps, const void* tail,
                    int64_t tail_slot_stride, int tail_cols, const int32_t* seqs, const int32_t* row_seq, int64_t rows, int dtype,
                    b200_stream_t stream) {
  B200_CHECK_ARG(in && groups && seqs && row_seq, "b200_short_conv: null pointer");
  B200_CHECK_ARG(n_groups >= 1 && n_groups <= kCvMaxGroups, "b200_short_conv: one to three groups");
  B200_CHECK_ARG(taps >= 1 && taps <= kCvMaxTaps + 1, "b200_short_conv: 1 to %d taps", kCvMaxTaps + 1);
  B200_CHECK_ARG(taps == 1 || tail, "b200_short_conv: a convolution over more than one tap needs the tail state");
  B200_CHECK_ARG(rows > 0 && rows <= 0x7fffffff, "b200_short_conv: bad row count");
  B200_CHECK_ARG((reinterpret_cast<uintptr_t>(seqs) & 15) == 0, "b200_short_conv: seqs must be 16-byte aligned");
  CvParams P{};
  P.n_groups = n_groups;
  P.taps = taps;
  for (int i = 0; i < n_groups; ++i) {
    const b200_conv_group& a = groups[i];
    B200_CHECK_ARG(a.w && a.out && a.heads > 0 && a.dim > 0 && a.dim <= 64 * kCvMaxIt, "b200_short_conv: bad group (head size up to %d)", 64 * kCvMaxIt);
    B200_CHECK_ARG(a.post != 1 || (a.rot_dims >= 0 && a.rot_dims <= a.dim && a.rot_dims % 2 == 0 && (a.rot_dims == 0 || a.inv_freq)),
                   "b200_short_conv: rotation needs an even number of dimensions and their frequencies");
    P.g[i] = CvGroup{a.w, a.out, a.ld_out, a.inv_freq, a.col0, a.heads, a.dim, a.act, a.post, a.rot_dims, a.out_f32, a.rot_mscale, a.post_scale, a.eps};
    P.total_heads += a.heads;
  }
  const int per = kCvThreads / 32;
  B200_CHECK_ARG((P.total_heads + per - 1) / per <= 65535, "b200_short_conv: too many heads");
  const dim3 grid((unsigned)rows, (unsigned)((P.total_heads + per - 1) / per));
  // pairs of neighbouring channels are read with one access when every head starts on an even channel of even-pitched, aligned rows
  const size_t esz = dtype == B200_F32 ? 4 : 2;
  int pairs = (ld_in % 2 == 0) && (tail_cols % 2 == 0) && (tail_slot_stride % 2 == 0) && (reinterpret_cast<uintptr_t>(in) % (2 * esz) == 0) &&
              (reinterpret_cast<uintptr_t>(tail) % (2 * esz) == 0);
  int max_dim = 0;
  bool w16 = true;
  for (int i = 0; i < n_groups; ++i) {
    pairs = pairs && groups[i].dim % 2 == 0 && groups[i].col0 % 2 == 0;
    w16 = w16 && reinterpret_cast<uintptr_t>(groups[i].w) % 16 == 0;
    max_dim = groups[i].dim > max_dim ? groups[i].dim : max_dim;
  }
  if (pairs && w16) pairs |= 2;   // even channels times four taps: every pair's taps start on a 16-byte boundary
  cudaStream_t st = (cudaStream_t)stream;
  const int4* sq = reinterpret_cast<const int4*>(seqs);
  B200_FLOAT_TYPES(dtype, T, {
    if (max_dim <= 64) B200_CUDA((short_conv_launch<T, 1>(taps, grid, st, (const T*)in, ld_in, P, (const T*)tail, tail_slot_stride, tail_cols, sq, row_seq, pairs)));
    else if (max_dim <= 128) B200_CUDA((short_conv_launch<T, 2>(taps, grid, st, (const T*)in, ld_in, P, (const T*)tail, tail_slot_stride, tail_cols, sq, row_seq, pairs)));
    else if (max_dim <= 256) B200_CUDA((short_conv_launch<T, 4>(taps, grid, st, (const T*)in, ld_in, P, (const T*)tail, tail_slot_stride, tail_cols, sq, row_seq, pairs)));
    else B200_CUDA((short_conv_launch<T, kCvMaxIt>(taps, grid, st, (const T*)in, ld_in, P, (const T*)tail, tail_slot_stride, tail_cols, sq, row_seq, pairs)));
  });
  return B200_OK;
}

int b200_conv_tail_update(const void* in, int64_t ld_in, void* tail, int64_t tail_slot_stride, int tail_cols, int taps, const int32_t* seqs,
                          int n_seqs, int dtype, b200_stream_t stream) {
  B200_CHECK_ARG(taps >= 1 && taps <= kCvMaxTaps + 1, "b200_conv_tail_update: 1 to %d taps", kCvMaxTaps + 1);
  if (taps == 1) return B200_OK;   // nothing is carried
  B200_CHECK_ARG(in && tail && seqs && n_seqs > 0 && n_seqs <= 65535 && tail_cols > 0, "b200_conv_tail_update: bad argument");
  B200_CHECK_ARG((reinterpret_cast<uintptr_t>(seqs) & 15) == 0, "b200_conv_tail_update: seqs must be 16-byte aligned");
  const dim3 grid((unsigned)((tail_cols + 255) / 256), (unsigned)n_seqs);
  B200_FLOAT_TYPES(dtype, T, B200_CUDA(launch(conv_tail_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)in, ld_in, (T*)tail,
                                               tail_slot_stride, tail_cols, taps, reinterpret_cast<const int4*>(seqs))));
  return B200_OK;
}

}  // extern "C"
