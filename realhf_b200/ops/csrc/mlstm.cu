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
//   mlstm_scan   one CTA per (sequence, head, chunk of columns).  A group of LPC lanes owns one column of the extended state with
//                32 rows per lane in registers; q / k / v / gates of 8 tokens are staged in shared memory (q, k as fp32, read back as
//                16-byte broadcasts); the lanes' partial dot products meet by shuffles.  The same kernel serves packed prompts
//                (state from zero or from the slot, left in the slot) and decode steps (sequences of one token).
//   mlstm_out    warp per (token, head): the denominator above, the head's RMS norm (no weight), then the full-width weight and
//                the sigmoid output gate.
#include "anytype.cuh"

namespace {

using rb::ld_any;
using rb::st_any;

constexpr int kThreads = 128, kTT = 8, kRPL = 32;

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
};

template <int LPC>
__global__ void __launch_bounds__(kThreads) mlstm_scan_kernel(ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int COLS = kThreads / LPC, DP = LPC * kRPL;
  float* qs = smem;                 // [kTT][DP]
  float* ks = qs + kTT * DP;        // [kTT][DP]
  float* vs = ks + kTT * DP;        // [kTT][COLS]
  float* gi = vs + kTT * COLS;      // [kTT]
  float* gf = gi + kTT;             // [kTT]
  const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int cl = tid / LPC, l = tid % LPC, col = blockIdx.z * COLS + cl;
  const int d = p.d, dv = p.dv, dvx = dv + 1, dt = p.dt;
  const bool active = col <= dv;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int s0 = p.cu ? p.cu[seq] : seq, L = p.cu ? p.cu[seq + 1] - s0 : 1;
  if (L <= 0) return;
  const int64_t slot = p.slots ? p.slots[seq] : seq;
  const int r0 = l * kRPL;
  float s[kRPL];
  float m = 0.f;
  float* Sg = p.S ? p.S + ((slot * p.H + h) * (int64_t)d) * dvx : nullptr;
  if (p.load_state && Sg != nullptr) {
#pragma unroll
    for (int r = 0; r < kRPL; ++r) s[r] = (active && r0 + r < d) ? Sg[(int64_t)(r0 + r) * dvx + col] : 0.f;
    m = p.M[slot * p.H + h];
  } else {
#pragma unroll
    for (int r = 0; r < kRPL; ++r) s[r] = 0.f;
  }
  const unsigned gmask = (LPC == 32) ? 0xffffffffu : (((1u << LPC) - 1u) << ((tid & 31) / LPC * LPC));
  for (int t0 = 0; t0 < L; t0 += kTT) {
    const int nt = min(kTT, L - t0);
    __syncthreads();
    for (int idx = tid; idx < nt * DP; idx += kThreads) {
      const int tt = idx / DP, e = idx % DP;
      const int64_t row = (int64_t)(s0 + t0 + tt) * p.ld;
      qs[idx] = e < d ? ld_any(p.proj, dt, row + h * d + e) * p.qscale : 0.f;
      ks[idx] = e < d ? ld_any(p.proj, dt, row + p.off_k + h * d + e) : 0.f;
    }
    for (int idx = tid; idx < nt * COLS; idx += kThreads) {
      const int tt = idx / COLS, c = blockIdx.z * COLS + idx % COLS;
      vs[idx] = c < dv ? ld_any(p.proj, dt, (int64_t)(s0 + t0 + tt) * p.ld + p.off_v + h * dv + c) : (c == dv ? 1.f : 0.f);
    }
    if (tid < nt) {
      const int64_t row = (int64_t)(s0 + t0 + tid) * p.ld + p.off_if;
      const float xi = ld_any(p.proj, dt, row + h) + ld_any(p.gate_bias, dt, h);
      const float xf = ld_any(p.proj, dt, row + p.H + h) + ld_any(p.gate_bias, dt, p.H + h);
      gi[tid] = p.cap * tanhf(xi / p.cap);
      const float z = p.cap * tanhf(xf / p.cap);
      gf[tid] = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float ig = gi[tt], fg = gf[tt];
      const float mn = fmaxf(fg + m, ig);
      const float dec = expf(fg + m - mn), inp = expf(ig - mn);
      m = mn;
      const float v = vs[tt * COLS + cl] * inp;
      const float* kr = ks + tt * DP + r0;
      const float* qr = qs + tt * DP + r0;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < kRPL; r += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(kr + r), qq = *reinterpret_cast<const float4*>(qr + r);
        s[r] = fmaf(dec, s[r], kk.x * v);         acc = fmaf(s[r], qq.x, acc);
        s[r + 1] = fmaf(dec, s[r + 1], kk.y * v); acc = fmaf(s[r + 1], qq.y, acc);
        s[r + 2] = fmaf(dec, s[r + 2], kk.z * v); acc = fmaf(s[r + 2], qq.z, acc);
        s[r + 3] = fmaf(dec, s[r + 3], kk.w * v); acc = fmaf(s[r + 3], qq.w, acc);
      }
#pragma unroll
      for (int o = LPC / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(gmask, acc, o, LPC);
      const int64_t t = s0 + t0 + tt;
      if (l == 0 && active) p.o[(t * p.H + h) * dvx + col] = acc;
      if (tid == 0 && blockIdx.z == 0) p.m_out[t * p.H + h] = m;
    }
  }
  if (Sg != nullptr) {
#pragma unroll
    for (int r = 0; r < kRPL; ++r)
      if (active && r0 + r < d) Sg[(int64_t)(r0 + r) * dvx + col] = s[r];
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

template <int LPC>
int launch_scan(const ScanParams& p, int n_seqs, cudaStream_t s) {
  constexpr int COLS = kThreads / LPC, DP = LPC * kRPL;
  const size_t smem = sizeof(float) * ((size_t)2 * kTT * DP + (size_t)kTT * COLS + 2 * kTT);
  auto kern = mlstm_scan_kernel<LPC>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
  dim3 grid((unsigned)n_seqs, (unsigned)p.H, (unsigned)RB_CEIL_DIV(p.dv + 1, COLS));
  return rb::launch_pdl(kern, grid, dim3(kThreads), smem, s, p) == cudaSuccess ? 0 : 2;
}

}  // namespace

// proj [T, ld] in type dt; o [T, H, dv + 1], m_out [T, H] fp32; cu null = decode step over n_seqs rows; S / M the slots' states
// (null: keep none).  load_state: start from the slot's state instead of zero.  Head sizes d up to 1024.
extern "C" int rb_mlstm_scan(const void* proj, int64_t ld, int dt, const void* gate_bias, float* o, float* m_out, const int* cu, float* S, float* M,
                             const int* slots, int n_seqs, int H, int d, int dv, int off_k, int off_v, int off_if, float cap, float qscale,
                             int load_state, cudaStream_t s) {
  if (n_seqs == 0) return 0;
  if (d < 1 || d > 32 * kRPL) return -1;
  ScanParams p{proj, ld, dt, gate_bias, o, m_out, cu, S, M, slots, H, d, dv, load_state, off_k, off_v, off_if, cap, qscale};
  const int lanes = RB_CEIL_DIV(d, kRPL);
  if (lanes <= 1) return launch_scan<1>(p, n_seqs, s);
  if (lanes <= 2) return launch_scan<2>(p, n_seqs, s);
  if (lanes <= 4) return launch_scan<4>(p, n_seqs, s);
  if (lanes <= 8) return launch_scan<8>(p, n_seqs, s);
  if (lanes <= 16) return launch_scan<16>(p, n_seqs, s);
  return launch_scan<32>(p, n_seqs, s);
}

extern "C" int rb_mlstm_out(const float* o, const float* m, const void* w, int dtw, const void* gate, int64_t ldg, int dtg, void* out, int dto,
                            int64_t T, int H, int dv, float eps, cudaStream_t s) {
  const int64_t rows = T * H;
  if (rows == 0) return 0;
  return rb::launch_pdl(mlstm_out_kernel, dim3((unsigned)RB_CEIL_DIV(rows, (int64_t)4)), dim3(128), 0, s, o, m, w, dtw, gate, ldg, dtg, out, dto, rows,
                        H, dv, eps) == cudaSuccess ? 0 : 2;
}
