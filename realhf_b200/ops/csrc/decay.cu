// Linear attention with a fixed decay per head (`DecayConfig`: retention, lightning attention) and the rotation of head vectors by
// their position.  Per head a matrix state S [d, dv] in fp32:
//
//   S_t = g_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t                         (no softmax, no denominator)
//
// Everything is fp32 arithmetic with exact sinf / cosf / expf (compiled without fast-math); storage types by a type code.
//
//   rotate_heads   in place, a CTA per token (its cos / sin table formed once in shared memory): the first `dims` dimensions of each of the n_h heads at the start of a row turn by
//                  angle = position * f_i (one fp32 product); pairs (i, i + dims / 2) or (2i, 2i + 1).  The position is pos[t], or in
//                  the step form lens[slot of row t].
//   decay_prepare  projection row [q (H d) | k (H d) | v (H dv) | ..] -> fp32 u [T, 2 H d + H dv]: SiLU on everything, or the rotation
//                  of q and k and a factor on k.
//   decay_scan     one CTA per (sequence, head, chunk of value columns).  A column of S depends only on its own value column, so a
//                  group of LPC lanes owns one or two columns with EPL rows per lane and column in registers.  The q, k and v of the next kTok tokens
//                  arrive by cp.async into the second of two shared-memory buffers while the current ones are consumed (one
//                  barrier per chunk); the lanes' partial dot products meet by shuffles.  The same kernel serves packed prompts
//                  (state from zero or from the slot, left in the slot) and decode steps (sequences of one token).
//   decay_out      one CTA per token: o / rms(o) per head, or over all heads times a weight; times silu or sigmoid of the gate.
#include "anytype.cuh"

namespace {

using rb::ld_any;
using rb::st_any;

RB_DEVICE int row_position(const int* pos, const int* lens, const int* slots, int64_t t) {
  if (pos != nullptr) return pos[t];
  return lens[slots != nullptr ? slots[t] : t];
}

// ------------------------------------------------------------------------------------------------ rotation in place
__global__ void __launch_bounds__(256) rotate_heads_kernel(void* __restrict__ x, int64_t ld, int dt, const int* __restrict__ pos,
                                                           const int* __restrict__ lens, const int* __restrict__ slots,
                                                           const float* __restrict__ inv_freq, int n_h, int d, int dims, int interleaved) {
  const int64_t t = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  const float p = (float)row_position(pos, lens, slots, t);
  const int half = dims / 2;
  for (int idx = threadIdx.x; idx < n_h * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const int64_t e0 = t * ld + (int64_t)h * d + (interleaved ? 2 * i : i), e1 = e0 + (interleaved ? 1 : half);
    float sn, cs;
    sincosf(p * inv_freq[i], &sn, &cs);
    const float u = ld_any(x, dt, e0), v = ld_any(x, dt, e1);
    st_any(x, dt, e0, u * cs - v * sn);
    st_any(x, dt, e1, v * cs + u * sn);
  }
}

// One CTA per token: the token's cos / sin table (dims / 2 entries) is formed once in shared memory, then every thread turns four
// consecutive elements per step (8- or 16-byte accesses): interleaved layout = two pairs inside the four; half layout = the four
// elements at i .. i + 3 of the first half with their partners in the second half.
constexpr int kMaxHalf = 512;

RB_DEVICE void fill_table(float* cs, float* sn, float p, const float* inv_freq, int half) {
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &sn[i], &cs[i]);
  __syncthreads();
}

__global__ void __launch_bounds__(256) rotate_heads_vec_kernel(void* __restrict__ x, int64_t ld, int dt, const int* __restrict__ pos,
                                                               const int* __restrict__ lens, const int* __restrict__ slots,
                                                               const float* __restrict__ inv_freq, int n_h, int d, int dims, int interleaved) {
  __shared__ float cs[kMaxHalf], sn[kMaxHalf];
  const int64_t t = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int half = dims / 2, per_head = (interleaved ? dims : half) / 4;
  fill_table(cs, sn, (float)row_position(pos, lens, slots, t), inv_freq, half);
  for (int r = threadIdx.x; r < n_h * per_head; r += blockDim.x) {
    const int h = r / per_head, c = (r - h * per_head) * 4;
    const int64_t e0 = t * ld + (int64_t)h * d + c;
    if (interleaved) {
      const float4 v = rb::ld4_any(x, dt, e0);
      const float c0 = cs[c / 2], s0 = sn[c / 2], c1 = cs[c / 2 + 1], s1 = sn[c / 2 + 1];
      rb::st4_any(x, dt, e0, make_float4(v.x * c0 - v.y * s0, v.y * c0 + v.x * s0, v.z * c1 - v.w * s1, v.w * c1 + v.z * s1));
    } else {
      const float4 u = rb::ld4_any(x, dt, e0), v = rb::ld4_any(x, dt, e0 + half);
      const float* k = cs + c;
      const float* m = sn + c;
      rb::st4_any(x, dt, e0, make_float4(u.x * k[0] - v.x * m[0], u.y * k[1] - v.y * m[1], u.z * k[2] - v.z * m[2], u.w * k[3] - v.w * m[3]));
      rb::st4_any(x, dt, e0 + half, make_float4(v.x * k[0] + u.x * m[0], v.y * k[1] + u.y * m[1], v.z * k[2] + u.z * m[2], v.w * k[3] + u.w * m[3]));
    }
  }
}

// ------------------------------------------------------------------------------------------------ prepare
RB_DEVICE float silu1(float x) { return x / (1.f + expf(-x)); }
RB_DEVICE float4 silu4(float4 v) { return make_float4(silu1(v.x), silu1(v.y), silu1(v.z), silu1(v.w)); }

// One CTA per token, four consecutive columns per thread and step, the cos / sin table in shared memory; a rotated group of four in
// the half layout also reads its partner group.
__global__ void __launch_bounds__(256) decay_prepare_vec_kernel(const void* __restrict__ proj, int64_t ld, int dt, float* __restrict__ u,
                                                                const int* __restrict__ pos, const int* __restrict__ lens,
                                                                const int* __restrict__ slots, const float* __restrict__ inv_freq, int H, int d,
                                                                int dv, int dims, int interleaved, int silu, float k_scale) {
  __shared__ float cs[kMaxHalf], sn[kMaxHalf];
  const int64_t t = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int nq = H * d, n = 2 * nq + H * dv, half = dims / 2;
  if (dims > 0) fill_table(cs, sn, (float)row_position(pos, lens, slots, t), inv_freq, half);
  const int64_t base = t * ld;
  for (int c = threadIdx.x * 4; c < n; c += blockDim.x * 4) {
    float4 x = rb::ld4_any(proj, dt, base + c);
    if (silu) x = silu4(x);
    if (c < 2 * nq) {
      const int e = c % d;
      if (e < dims) {
        if (interleaved) {
          const float c0 = cs[e / 2], s0 = sn[e / 2], c1 = cs[e / 2 + 1], s1 = sn[e / 2 + 1];
          x = make_float4(x.x * c0 - x.y * s0, x.y * c0 + x.x * s0, x.z * c1 - x.w * s1, x.w * c1 + x.z * s1);
        } else {
          const bool first = e < half;
          const int i = first ? e : e - half;
          float4 y = rb::ld4_any(proj, dt, base + (first ? c + half : c - half));
          if (silu) y = silu4(y);
          const float* k = cs + i;
          const float* m = sn + i;
          x = first ? make_float4(x.x * k[0] - y.x * m[0], x.y * k[1] - y.y * m[1], x.z * k[2] - y.z * m[2], x.w * k[3] - y.w * m[3])
                    : make_float4(x.x * k[0] + y.x * m[0], x.y * k[1] + y.y * m[1], x.z * k[2] + y.z * m[2], x.w * k[3] + y.w * m[3]);
        }
      }
      if (c >= nq) x = make_float4(x.x * k_scale, x.y * k_scale, x.z * k_scale, x.w * k_scale);
    }
    *reinterpret_cast<float4*>(u + t * (int64_t)n + c) = x;
  }
}

__global__ void __launch_bounds__(256) decay_prepare_kernel(const void* __restrict__ proj, int64_t ld, int dt, float* __restrict__ u,
                                                            const int* __restrict__ pos, const int* __restrict__ lens,
                                                            const int* __restrict__ slots, const float* __restrict__ inv_freq, int H, int d,
                                                            int dv, int dims, int interleaved, int silu, float k_scale) {
  const int64_t t = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int nq = H * d, n = 2 * nq + H * dv, half = dims / 2;
  const float p = dims > 0 ? (float)row_position(pos, lens, slots, t) : 0.f;
  const int64_t base = t * ld;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float x = ld_any(proj, dt, base + c);
    if (silu) x = x / (1.f + expf(-x));
    if (c < 2 * nq) {
      const int e = c % d;
      if (e < dims) {
        // partner of the pair and the sign of the sine term: (u, v) -> (u cos - v sin, v cos + u sin)
        int i, partner;
        bool first;
        if (interleaved) { i = e >> 1; first = (e & 1) == 0; partner = first ? c + 1 : c - 1; }
        else { first = e < half; i = first ? e : e - half; partner = first ? c + half : c - half; }
        float y = ld_any(proj, dt, base + partner);
        if (silu) y = y / (1.f + expf(-y));
        float sn, cs;
        sincosf(p * inv_freq[i], &sn, &cs);
        x = first ? x * cs - y * sn : x * cs + y * sn;
      }
      if (c >= nq) x *= k_scale;
    }
    u[t * (int64_t)n + c] = x;
  }
}

// ------------------------------------------------------------------------------------------------ scan
constexpr int kThreads = 128;
constexpr int scan_tokens(int dp) { return dp <= 128 ? 8 : (dp <= 512 ? 4 : 2); }

struct ScanParams {
  const float* u; int64_t ld;             // [T, ld] = [q (H d) | k (H d) | v (H dv)]
  const float* decay;                     // [H]
  float* o;                               // [T, H, dv]
  const int* cu;                          // [n_seqs + 1]; null: sequence b is row b alone (decode step)
  float* S;                               // [n_slots, H, d, dv] or null
  const int* slots;                       // [n_seqs] or null (sequence b = slot b)
  int H, d, dv, load_state;
  int vec;                                // rows allow 16-byte copies (d, dv, ld multiples of 4, u 16-byte aligned)
};

RB_DEVICE void cp_async4(float* dst, const float* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(src) : "memory");
}
RB_DEVICE void cp_async16(float* dst, const float* src) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(src) : "memory");
}
RB_DEVICE void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
RB_DEVICE void cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int LPC, int EPL, int CPT>
__global__ void __launch_bounds__(kThreads, EPL * CPT == 32 ? 3 : 2) decay_scan_kernel(ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int NCOL = kThreads / LPC * CPT, DP = LPC * EPL, kTok = scan_tokens(DP);
  constexpr int kBuf = kTok * (2 * DP + NCOL);                     // floats of one staging buffer: q, k, v of kTok tokens
  const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, c0 = blockIdx.z * NCOL;
  const int l = tid % LPC, cl = (tid / LPC) * CPT;                 // this thread's first column inside the CTA's chunk
  const int d = p.d, dv = p.dv;
  const int col = c0 + cl;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int t0 = p.cu ? p.cu[seq] : seq, t1 = p.cu ? p.cu[seq + 1] : seq + 1;
  if (t1 <= t0) return;
  const int64_t slot = p.slots ? p.slots[seq] : seq;
  const float g = p.decay[h];
  // lane l of a column group owns rows ((e / 4) * LPC + l) * 4 + e % 4: float4 reads of k and q from shared memory without bank
  // conflicts, each reused for the thread's CPT columns
  auto row_of = [&](int e) { return ((e >> 2) * LPC + l) * 4 + (e & 3); };
  float S[CPT][EPL];
  float* Sg = p.S ? p.S + ((slot * p.H + h) * (int64_t)d) * dv : nullptr;
  const bool load = p.load_state && Sg != nullptr;
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const int row = row_of(e);
      S[c][e] = (load && col + c < dv && row < d) ? Sg[(int64_t)row * dv + col + c] : 0.f;
    }
  // the padding rows d .. DP of the q / k staging rows and the columns beyond dv are never written by cp.async: zero both buffers once
  for (int idx = tid; idx < 2 * kBuf; idx += kThreads) smem[idx] = 0.f;
  __syncthreads();
  auto fetch = [&](float* buf, int tb) {
    const int nt = min(kTok, t1 - tb);
    if (p.vec) {
      const int d4 = d >> 2;
      for (int idx = tid; idx < nt * d4; idx += kThreads) {
        const int tt = idx / d4, e = (idx - tt * d4) * 4;
        const float* src = p.u + (int64_t)(tb + tt) * p.ld + h * d + e;
        cp_async16(buf + tt * DP + e, src);
        cp_async16(buf + kTok * DP + tt * DP + e, src + p.H * d);
      }
      for (int idx = tid; idx < nt * (NCOL / 4); idx += kThreads) {
        const int tt = idx / (NCOL / 4), c = (idx - tt * (NCOL / 4)) * 4;
        if (c0 + c < dv) cp_async16(buf + 2 * kTok * DP + tt * NCOL + c, p.u + (int64_t)(tb + tt) * p.ld + 2 * p.H * d + h * dv + c0 + c);
      }
      cp_commit();
      return;
    }
    for (int idx = tid; idx < nt * d; idx += kThreads) {
      const int tt = idx / d, e = idx - tt * d;
      const float* src = p.u + (int64_t)(tb + tt) * p.ld + h * d + e;
      cp_async4(buf + tt * DP + e, src);
      cp_async4(buf + kTok * DP + tt * DP + e, src + p.H * d);
    }
    for (int idx = tid; idx < nt * NCOL; idx += kThreads) {
      const int tt = idx / NCOL, c = idx - tt * NCOL;
      if (c0 + c < dv) cp_async4(buf + 2 * kTok * DP + tt * NCOL + c, p.u + (int64_t)(tb + tt) * p.ld + 2 * p.H * d + h * dv + c0 + c);
    }
    cp_commit();
  };
  fetch(smem, t0);
  int which = 0;
  for (int tb = t0; tb < t1; tb += kTok, which ^= 1) {
    const int nt = min(kTok, t1 - tb);
    float* buf = smem + which * kBuf;
    cp_wait_all();
    __syncthreads();                       // this chunk has landed for every thread; the other buffer is no longer read
    if (tb + kTok < t1) fetch(smem + (which ^ 1) * kBuf, tb + kTok);
    const float* qs = buf;
    const float* ks = buf + kTok * DP;
    const float* vs = ks + kTok * DP;
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      float v[CPT], a[CPT][4];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        v[c] = vs[tt * NCOL + cl + c];
        a[c][0] = a[c][1] = a[c][2] = a[c][3] = 0.f;
      }
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DP) + l;
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DP) + l;
#pragma unroll
      for (int e4 = 0; e4 < EPL / 4; ++e4) {
        const float4 kk = k4[e4 * LPC], qq = q4[e4 * LPC];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          S[c][e4 * 4] = fmaf(g, S[c][e4 * 4], kk.x * v[c]);         a[c][0] = fmaf(S[c][e4 * 4], qq.x, a[c][0]);
          S[c][e4 * 4 + 1] = fmaf(g, S[c][e4 * 4 + 1], kk.y * v[c]); a[c][1] = fmaf(S[c][e4 * 4 + 1], qq.y, a[c][1]);
          S[c][e4 * 4 + 2] = fmaf(g, S[c][e4 * 4 + 2], kk.z * v[c]); a[c][2] = fmaf(S[c][e4 * 4 + 2], qq.z, a[c][2]);
          S[c][e4 * 4 + 3] = fmaf(g, S[c][e4 * 4 + 3], kk.w * v[c]); a[c][3] = fmaf(S[c][e4 * 4 + 3], qq.w, a[c][3]);
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        float acc = (a[c][0] + a[c][1]) + (a[c][2] + a[c][3]);
#pragma unroll
        for (int off = 1; off < LPC; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (l == 0 && col + c < dv) p.o[((int64_t)(tb + tt) * p.H + h) * dv + col + c] = acc;
      }
    }
  }
  if (Sg != nullptr) {
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int row = row_of(e);
        if (col + c < dv && row < d) Sg[(int64_t)row * dv + col + c] = S[c][e];
      }
  }
}

template <int LPC, int EPL, int CPT>
int launch_scan(const ScanParams& p, int n_seqs, cudaStream_t s) {
  constexpr int NCOL = kThreads / LPC * CPT, DP = LPC * EPL, kTok = scan_tokens(DP);
  const size_t smem = sizeof(float) * 2 * (size_t)kTok * (2 * DP + NCOL);
  auto kern = decay_scan_kernel<LPC, EPL, CPT>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
  dim3 grid((unsigned)n_seqs, (unsigned)p.H, (unsigned)RB_CEIL_DIV(p.dv, NCOL));
  return rb::launch_pdl(kern, grid, dim3(kThreads), smem, s, p) == cudaSuccess ? 0 : 2;
}

// ------------------------------------------------------------------------------------------------ output norm and gate
template <bool kVec>
__global__ void __launch_bounds__(128) decay_out_kernel(const float* __restrict__ o, const void* __restrict__ w, int dtw, const void* __restrict__ gate,
                                                        int64_t ldg, int dtg, void* __restrict__ out, int dto, int H, int dv, float eps, int full,
                                                        int silu) {
  __shared__ float red[32];
  __shared__ float s_r;
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n = H * dv;
  rb::pdl_trigger();
  rb::pdl_wait();
  const float* orow = o + t * (int64_t)n;
  auto act = [&](float gv) {
    const float sg = 1.f / (1.f + expf(-gv));
    return silu ? gv * sg : sg;
  };
  auto emit = [&](int c, float r) {               // kVec: the four elements c .. c + 3
    if constexpr (kVec) {
      const float4 ov = *reinterpret_cast<const float4*>(orow + c), gv = rb::ld4_any(gate, dtg, t * ldg + c);
      float4 y = make_float4(ov.x * r, ov.y * r, ov.z * r, ov.w * r);
      if (w != nullptr) { const float4 wv = rb::ld4_any(w, dtw, c); y = make_float4(y.x * wv.x, y.y * wv.y, y.z * wv.z, y.w * wv.w); }
      rb::st4_any(out, dto, t * (int64_t)n + c, make_float4(y.x * act(gv.x), y.y * act(gv.y), y.z * act(gv.z), y.w * act(gv.w)));
    } else {
      float y = orow[c] * r;
      if (w != nullptr) y *= ld_any(w, dtw, c);
      st_any(out, dto, t * (int64_t)n + c, y * act(ld_any(gate, dtg, t * ldg + c)));
    }
  };
  auto sumsq = [&](int c) {
    if constexpr (kVec) {
      const float4 v = *reinterpret_cast<const float4*>(orow + c);
      return (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    } else {
      return orow[c] * orow[c];
    }
  };
  constexpr int V = kVec ? 4 : 1;
  if (full) {
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < n; c += blockDim.x * V) ss += sumsq(c);
    ss = rb::block_reduce<false>(ss, red);
    if (threadIdx.x == 0) s_r = 1.f / sqrtf(ss / (float)n + eps);
    __syncthreads();
    const float r = s_r;
    for (int c = threadIdx.x * V; c < n; c += blockDim.x * V) emit(c, r);
    return;
  }
  for (int h = warp; h < H; h += 4) {
    float ss = 0.f;
    for (int c = lane * V; c < dv; c += 32 * V) ss += sumsq(h * dv + c);
    ss = rb::warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)dv + eps);
    for (int c = lane * V; c < dv; c += 32 * V) emit(h * dv + c, r);
  }
}

}  // namespace

extern "C" {

int rb_rotate_heads(void* x, int64_t ld, int dt, const int* pos, const int* lens, const int* slots, const float* inv_freq, int64_t T, int n_h, int d,
                    int dims, int interleaved, cudaStream_t s) {
  if (T == 0 || dims == 0) return 0;
  if (dims % 2 || dims > d || (pos == nullptr && lens == nullptr)) return -1;
  const int grp = (interleaved ? dims : dims / 2);
  if (d % 4 == 0 && grp % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && dims / 2 <= kMaxHalf)
    return rb::launch_pdl(rotate_heads_vec_kernel, dim3((unsigned)T), dim3(256), 0, s, x, ld, dt, pos, lens, slots, inv_freq, n_h, d, dims,
                          interleaved) == cudaSuccess ? 0 : 2;
  return rb::launch_pdl(rotate_heads_kernel, dim3((unsigned)T), dim3(256), 0, s, x, ld, dt, pos, lens, slots, inv_freq, n_h, d, dims,
                        interleaved) == cudaSuccess ? 0 : 2;
}

int rb_decay_prepare(const void* proj, int64_t ld, int dt, float* u, const int* pos, const int* lens, const int* slots, const float* inv_freq,
                     int64_t T, int H, int d, int dv, int dims, int interleaved, int silu, float k_scale, cudaStream_t s) {
  if (T == 0) return 0;
  if (dims % 2 || dims > d || (dims > 0 && ((pos == nullptr && lens == nullptr) || inv_freq == nullptr))) return -1;
  const int grp = (interleaved ? dims : dims / 2);
  if (d % 4 == 0 && dv % 4 == 0 && grp % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(u) & 15) == 0 && dims / 2 <= kMaxHalf)
    return rb::launch_pdl(decay_prepare_vec_kernel, dim3((unsigned)T), dim3(256), 0, s, proj, ld, dt, u, pos, lens, slots, inv_freq, H, d, dv, dims,
                          interleaved, silu, k_scale) == cudaSuccess ? 0 : 2;
  return rb::launch_pdl(decay_prepare_kernel, dim3((unsigned)T), dim3(256), 0, s, proj, ld, dt, u, pos, lens, slots, inv_freq, H, d, dv, dims,
                        interleaved, silu, k_scale) == cudaSuccess ? 0 : 2;
}

// u [T, ld] fp32; o [T, H, dv] fp32; cu null = decode step over n_seqs rows; S the slots' states (null: keep none).  load_state:
// start from the slot's state instead of zero.  Head sizes d up to 1024.
int rb_decay_scan(const float* u, int64_t ld, const float* decay, float* o, const int* cu, float* S, const int* slots, int n_seqs, int H, int d,
                  int dv, int load_state, cudaStream_t s) {
  if (n_seqs == 0) return 0;
  if (d < 1 || d > 1024 || dv < 1) return -1;
  const int vec = d % 4 == 0 && dv % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(u) & 15) == 0;
  ScanParams p{u, ld, decay, o, cu, S, slots, H, d, dv, load_state, vec};
  // (lanes per column group, state rows per lane, columns per thread): 64 state registers per thread from d = 64 on; two columns per
  // thread halve the shared-memory reads of q and k per multiply-add (d = 128: 1.93 -> 1.60 ms for 32 x 1024 tokens x 16 heads)
  if (d <= 32) return launch_scan<1, 32, 1>(p, n_seqs, s);
  if (d <= 64) return launch_scan<2, 32, 2>(p, n_seqs, s);
  if (d <= 128) return launch_scan<4, 32, 2>(p, n_seqs, s);   // (four columns x 16 rows per lane: no faster, 1.64 ms)
  if (d <= 256) return launch_scan<8, 32, 2>(p, n_seqs, s);
  if (d <= 512) return launch_scan<16, 32, 2>(p, n_seqs, s);
  return launch_scan<32, 32, 2>(p, n_seqs, s);
}

int rb_decay_out(const float* o, const void* w, int dtw, const void* gate, int64_t ldg, int dtg, void* out, int dto, int64_t T, int H, int dv,
                 float eps, int full, int silu, cudaStream_t s) {
  if (T == 0) return 0;
  auto al = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec = dv % 4 == 0 && ldg % 4 == 0 && al(o) && al(w) && al(gate) && al(out);
  return rb::launch_pdl(vec ? decay_out_kernel<true> : decay_out_kernel<false>, dim3((unsigned)T), dim3(128), 0, s, o, w, dtw, gate, ldg, dtg, out,
                        dto, H, dv, eps, full, silu) == cudaSuccess ? 0 : 2;
}

}  // extern "C"
