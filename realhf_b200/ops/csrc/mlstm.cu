// Matrix-memory LSTM (`MLSTMConfig`): per head a matrix state S [d, dv], a normaliser n [d] and a running maximum m of the log
// gates, all fp32:
//
//   i_t = cap tanh((x_i + b_i) / cap)                       log input gate
//   f_t = logsigmoid(cap tanh((x_f + b_f) / cap))           log forget gate
//   m_t = max(f_t + m_(t-1), i_t)                           (m starts at 0)
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t the same with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// n is carried as one more column of S (a value that is always 1), so the state of a head is [d, dv + 1] and the kernel's raw
// output row is [S^T q | n . q].
//
//   mlstm_scan   one CTA per (sequence, head, chunk of columns).  A column of the extended state depends only on its own value
//                column, so columns are independent: a group of LPC lanes owns one column with EPL (32 or 64) rows per lane in
//                registers, and a CTA of four warps 128 / LPC value columns; the first warp of a head's first CTA also carries
//                the normaliser (DP / 32 rows per lane).  q, k, v and the gates of the next chunk of tokens are fetched into registers (16-byte loads
//                where the rows allow it) while the current chunk is processed out of shared memory (two staging buffers, one
//                barrier per chunk; q, k staged as fp32 and read back as 16-byte broadcasts); the lanes' partial dot products meet
//                by shuffles.  The same kernel serves packed prompts (state from zero or from the slot, left in the slot) and
//                decode steps (sequences of one token).
//   mlstm_out    warp per (token, head): the denominator above, the head's RMS norm (no weight), then the full-width weight and
//                the sigmoid output gate.
#include "anytype.cuh"

namespace {

using rb::ld_any;
using rb::st_any;

constexpr int kThreads = 128;

struct ScanParams {
  const void* proj; int64_t ld; int dt;   // [T, ld] = [q (H d) | k (H d) | v (H dv) | ... | x_i (H), x_f (H)] at the offsets below
  const void* gate_bias;                  // [2 H] = b_i, b_f in the model type
  float* o;                               // [T, H, dv + 1]
  float* m_out;                           // [T, H]
  const int* cu;                          // [n_seqs + 1]; null: sequence b is row b alone (decode step)
  float* S;                               // [n_slots, H, d, dv + 1] or null
  float* M;                               // [n_slots, H]
  const int* slots;                       // [n_seqs] or null (sequence b = slot b)
  int H, d, dv, load_state, off_k, off_v, off_if;
  float cap, qscale;
  int vec;                                // q / k rows can be read 16 bytes at a time
};

template <typename T> struct Unpack;
template <> struct Unpack<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void to(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
};
template <> struct Unpack<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void to(const uint4& r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};
template <> struct Unpack<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void to(const uint4& r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&w[i])); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
  }
};

// tokens per staged chunk: the prefetch of a chunk's q and k stays within a few 16-byte registers per thread
constexpr int chunk_tokens(int dpad) { return dpad <= 256 ? 8 : (dpad <= 512 ? 4 : 2); }

template <typename T, int LPC, int EPL>
__global__ void __launch_bounds__(kThreads, EPL == 32 ? 3 : 2) mlstm_scan_kernel(ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int NCOL = kThreads / LPC, DP = LPC * EPL, kTok = chunk_tokens(DP);
  constexpr int kBuf = 2 * kTok * DP + kTok * NCOL + 2 * kTok;       // floats of one staging buffer: q, k, v, (i, f)
  constexpr int N = Unpack<T>::N, VPR = DP / N, VQ = kTok * VPR;      // elements per 16-byte load, loads per staged row / chunk
  constexpr int NQV = (VQ + kThreads - 1) / kThreads, NV = (kTok * NCOL + kThreads - 1) / kThreads;
  const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, c0 = blockIdx.z * NCOL;
  constexpr int NR = DP / 32;                                          // normaliser rows per lane: j * 32 + lane
  const bool norm_warp = tid < 32 && blockIdx.z == 0;                  // this warp also carries the normaliser column (v = 1)
  const int l = tid % LPC, cl = tid / LPC, lane = tid & 31;
  const int d = p.d, dv = p.dv, dvx = dv + 1, dt = p.dt;
  const int col = c0 + cl;
  const bool active = col < dv;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int t0 = p.cu ? p.cu[seq] : seq, t1 = p.cu ? p.cu[seq + 1] : seq + 1;
  if (t1 <= t0) return;
  const int64_t slot = p.slots ? p.slots[seq] : seq;
  auto row_of = [&](int e) { return ((e >> 2) * LPC + l) * 4 + (e & 3); };
  float S[EPL];
  float m = 0.f;
  float* Sg = p.S ? p.S + ((slot * p.H + h) * (int64_t)d) * dvx : nullptr;
  const bool load = p.load_state && Sg != nullptr;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const int row = row_of(e);
    S[e] = (load && active && row < d) ? Sg[(int64_t)row * dvx + col] : 0.f;
  }
  float nrm[NR];
#pragma unroll
  for (int j = 0; j < NR; ++j) nrm[j] = (load && norm_warp && j * 32 + lane < d) ? Sg[(int64_t)(j * 32 + lane) * dvx + dv] : 0.f;
  if (load) m = p.M[slot * p.H + h];

  uint4 rq[NQV], rk[NQV];
  float rv[NV], rg = 0.f;
  auto fetch = [&](int tb) {
    const int nt = min(kTok, t1 - tb);
    if (p.vec) {
      const T* src = static_cast<const T*>(p.proj);
#pragma unroll
      for (int i = 0; i < NQV; ++i) {
        const int vi = tid + i * kThreads, tt = vi / VPR, e = (vi % VPR) * N;
        rq[i] = rk[i] = make_uint4(0u, 0u, 0u, 0u);
        if (vi < VQ && tt < nt && e < d) {
          const T* row = src + (int64_t)(tb + tt) * p.ld + h * d + e;
          rq[i] = *reinterpret_cast<const uint4*>(row);
          rk[i] = *reinterpret_cast<const uint4*>(row + p.off_k);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = tid + i * kThreads, tt = idx / NCOL, c = c0 + idx % NCOL;
      rv[i] = (idx < kTok * NCOL && tt < nt && c < dv) ? ld_any(p.proj, dt, (int64_t)(tb + tt) * p.ld + p.off_v + h * dv + c) : 0.f;
    }
    const int gt = kThreads - 1 - tid;                                 // the last warp brings the gates: (token, i or f)
    if (gt < 2 * nt)
      rg = ld_any(p.proj, dt, (int64_t)(tb + gt / 2) * p.ld + p.off_if + (gt & 1) * p.H + h) + ld_any(p.gate_bias, dt, (gt & 1) * p.H + h);
  };
  auto stage = [&](float* buf, int tb) {
    float* qs = buf;
    float* ks = buf + kTok * DP;
    if (p.vec) {
#pragma unroll
      for (int i = 0; i < NQV; ++i) {
        const int vi = tid + i * kThreads;
        if (vi < VQ) {
          float fq[N], fk[N];
          Unpack<T>::to(rq[i], fq);
          Unpack<T>::to(rk[i], fk);
#pragma unroll
          for (int j = 0; j < N; j += 4) {
            *reinterpret_cast<float4*>(qs + vi * N + j) = make_float4(fq[j] * p.qscale, fq[j + 1] * p.qscale, fq[j + 2] * p.qscale, fq[j + 3] * p.qscale);
            *reinterpret_cast<float4*>(ks + vi * N + j) = make_float4(fk[j], fk[j + 1], fk[j + 2], fk[j + 3]);
          }
        }
      }
    } else {                                                           // rows that allow no 16-byte loads: fetched here
      const int nt = min(kTok, t1 - tb);
      for (int idx = tid; idx < kTok * DP; idx += kThreads) {
        const int tt = idx / DP, e = idx % DP;
        const bool ok = tt < nt && e < d;
        const int64_t row = (int64_t)(tb + tt) * p.ld;
        qs[idx] = ok ? ld_any(p.proj, dt, row + h * d + e) * p.qscale : 0.f;
        ks[idx] = ok ? ld_any(p.proj, dt, row + p.off_k + h * d + e) : 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (tid + i * kThreads < kTok * NCOL) buf[2 * kTok * DP + tid + i * kThreads] = rv[i];
    const int gt = kThreads - 1 - tid;
    if (gt < 2 * kTok) {
      const float z = p.cap * tanhf(rg / p.cap);
      buf[2 * kTok * DP + kTok * NCOL + gt] = (gt & 1) ? fminf(z, 0.f) - log1pf(expf(-fabsf(z))) : z;
    }
  };

  fetch(t0);
  int which = 0;
  for (int tb = t0; tb < t1; tb += kTok, which ^= 1) {
    const int nt = min(kTok, t1 - tb);
    float* buf = smem + which * kBuf;
    stage(buf, tb);
    __syncthreads();
    if (tb + kTok < t1) fetch(tb + kTok);
    const float* qs = buf;
    const float* ks = buf + kTok * DP;
    const float* vs = ks + kTok * DP;
    const float* gs = vs + kTok * NCOL;
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const float ig = gs[tt * 2], fg = gs[tt * 2 + 1];
      const float mn = fmaxf(fg + m, ig);
      const float dec = expf(fg + m - mn), inp = expf(ig - mn);
      m = mn;
      const float v = vs[tt * NCOL + cl] * inp;
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DP) + l;
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DP) + l;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int e4 = 0; e4 < EPL / 4; ++e4) {
        const float4 kk = k4[e4 * LPC], qq = q4[e4 * LPC];
        S[e4 * 4] = fmaf(dec, S[e4 * 4], kk.x * v);         a0 = fmaf(S[e4 * 4], qq.x, a0);
        S[e4 * 4 + 1] = fmaf(dec, S[e4 * 4 + 1], kk.y * v); a1 = fmaf(S[e4 * 4 + 1], qq.y, a1);
        S[e4 * 4 + 2] = fmaf(dec, S[e4 * 4 + 2], kk.z * v); a2 = fmaf(S[e4 * 4 + 2], qq.z, a2);
        S[e4 * 4 + 3] = fmaf(dec, S[e4 * 4 + 3], kk.w * v); a3 = fmaf(S[e4 * 4 + 3], qq.w, a3);
      }
      float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
      for (int off = 1; off < LPC; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      const int64_t t = tb + tt;
      if (l == 0 && active) p.o[(t * p.H + h) * dvx + col] = acc;
      if (norm_warp) {
        float nq = 0.f;
#pragma unroll
        for (int j = 0; j < NR; ++j) {
          nrm[j] = fmaf(dec, nrm[j], ks[tt * DP + j * 32 + lane] * inp);
          nq = fmaf(nrm[j], qs[tt * DP + j * 32 + lane], nq);
        }
        nq = rb::warp_sum(nq);
        if (lane == 0) p.o[(t * p.H + h) * dvx + dv] = nq;
      }
      if (tid == 0 && blockIdx.z == 0) p.m_out[t * p.H + h] = m;
    }
  }
  if (Sg != nullptr) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int row = row_of(e);
      if (active && row < d) Sg[(int64_t)row * dvx + col] = S[e];
    }
    if (norm_warp) {
#pragma unroll
      for (int j = 0; j < NR; ++j)
        if (j * 32 + lane < d) Sg[(int64_t)(j * 32 + lane) * dvx + dv] = nrm[j];
    }
    if (tid == 0 && blockIdx.z == 0) p.M[slot * p.H + h] = m;
  }
}

// 4 warps per CTA, a warp per (token, head)
__global__ void __launch_bounds__(128) mlstm_out_kernel(const float* __restrict__ o, const float* __restrict__ m, const void* __restrict__ w, int dtw,
                                                        const void* __restrict__ gate, int64_t ldg, int dtg, void* __restrict__ out, int dto,
                                                        int64_t n_rows, int H, int dv, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);   // (token, head)
  rb::pdl_trigger();
  rb::pdl_wait();
  if (row >= n_rows) return;
  const int64_t t = row / H;
  const int h = (int)(row % H);
  const float* orow = o + row * (dv + 1);
  const float den = fmaxf(fabsf(orow[dv]), expf(-m[row])) + 1e-6f;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) { const float y = orow[c] / den; ss += y * y; }
  ss = rb::warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float g = ld_any(gate, dtg, t * ldg + h * dv + c);
    st_any(out, dto, t * (int64_t)(H * dv) + h * dv + c, orow[c] / den * r * ld_any(w, dtw, h * dv + c) * (1.f / (1.f + expf(-g))));
  }
}

template <typename T, int LPC, int EPL>
int launch_scan_t(const ScanParams& p, int n_seqs, cudaStream_t s) {
  constexpr int NCOL = kThreads / LPC, DP = LPC * EPL, kTok = chunk_tokens(DP);
  const size_t smem = sizeof(float) * 2 * ((size_t)2 * kTok * DP + (size_t)kTok * NCOL + 2 * kTok);
  auto kern = mlstm_scan_kernel<T, LPC, EPL>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
  dim3 grid((unsigned)n_seqs, (unsigned)p.H, (unsigned)RB_CEIL_DIV(p.dv, NCOL));
  return rb::launch_pdl(kern, grid, dim3(kThreads), smem, s, p) == cudaSuccess ? 0 : 2;
}

template <int LPC, int EPL>
int launch_scan(const ScanParams& p, int n_seqs, cudaStream_t s) {
  if (p.dt == 0) return launch_scan_t<float, LPC, EPL>(p, n_seqs, s);
  if (p.dt == 1) return launch_scan_t<__nv_bfloat16, LPC, EPL>(p, n_seqs, s);
  return launch_scan_t<__half, LPC, EPL>(p, n_seqs, s);
}

}  // namespace

// proj [T, ld] in type dt; o [T, H, dv + 1], m_out [T, H] fp32; cu null = decode step over n_seqs rows; S / M the slots' states
// (null: keep none).  load_state: start from the slot's state instead of zero.  Head sizes d up to 1024.
extern "C" int rb_mlstm_scan(const void* proj, int64_t ld, int dt, const void* gate_bias, float* o, float* m_out, const int* cu, float* S, float* M,
                             const int* slots, int n_seqs, int H, int d, int dv, int off_k, int off_v, int off_if, float cap, float qscale,
                             int load_state, cudaStream_t s) {
  if (n_seqs == 0) return 0;
  if (d < 1 || d > 1024 || dv < 1) return -1;
  const int n16 = dt == 0 ? 4 : 8;
  const int vec = d % n16 == 0 && ld % n16 == 0 && off_k % n16 == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0;
  ScanParams p{proj, ld, dt, gate_bias, o, m_out, cu, S, M, slots, H, d, dv, load_state, off_k, off_v, off_if, cap, qscale, vec};
  if (d <= 32) return launch_scan<1, 32>(p, n_seqs, s);
  if (d <= 64) return launch_scan<2, 32>(p, n_seqs, s);
  if (d <= 128) return launch_scan<2, 64>(p, n_seqs, s);
  if (d <= 256) return launch_scan<4, 64>(p, n_seqs, s);
  if (d <= 512) return launch_scan<8, 64>(p, n_seqs, s);
  return launch_scan<16, 64>(p, n_seqs, s);
}

extern "C" int rb_mlstm_out(const float* o, const float* m, const void* w, int dtw, const void* gate, int64_t ldg, int dtg, void* out, int dto,
                            int64_t T, int H, int dv, float eps, cudaStream_t s) {
  const int64_t rows = T * H;
  if (rows == 0) return 0;
  return rb::launch_pdl(mlstm_out_kernel, dim3((unsigned)RB_CEIL_DIV(rows, (int64_t)4)), dim3(128), 0, s, o, m, w, dtw, gate, ldg, dtg, out, dto, rows,
                        H, dv, eps) == cudaSuccess ? 0 : 2;
}
