// Latent attention with a rotated key part (`LatentAttentionConfig` with `rot_dim` > 0): the row a token leaves in the cache is
// [c | k_rot], c = RMSNorm(latent) * w of rank r and k_rot the rotated `rot` last outputs of the down-projection, shared by all
// heads.  Queries may pass a normalised latent of their own (q_rank > 0).  Rotation: pair (2i, 2i + 1) turns by the angle
// pos * f_i (fp32 product, sincosf), cos and sin times `mscale`; the frequency table f (with any rescaling of long contexts already
// applied) comes from the host.  All arithmetic is fp32; storage types by run-time code (anytype.cuh).
//
//   latent_rope_prepare    one CTA per token: cq = RMSNorm(proj[:, :q_rank]) * w_q -> [T, q_rank]; [c | k_rot] -> packed
//                          [T, r + rot] and / or the ring cache.  Packed form: position pos[t], cache row written when the token is
//                          among the last R of its sequence; step form: position lens[slot].
//   latent_rope_assemble   one CTA per token: q [T, H (d + rot)] with its rotated part turned, and per head the key
//                          [k_nope_h | k_rot] -> one tensor [T, 2 H (d + rot)] = [queries | keys] for the packed attention kernel.
//   latent_query_rope      decode: scale * rotate(q_rot) -> columns [r, r + rot) of the absorbed query [H, B, r + rot] fp32.
//   sigmoid_gate_          out[t, c] *= sigmoid(g[t, c]).
#include "anytype.cuh"

namespace {

using rb::ld_any;
using rb::st_any;

struct PrepParams {
  const void* proj; int64_t ld; int dt;
  const void* wq; const void* wc;          // norm weights [q_rank], [r]
  const float* inv_freq; float mscale;
  const int* pos;                          // packed form: [T]; null = step form
  const int* lens; const int* slots;       // step form: position = lens[slot], slot = slots ? slots[t] : t
  const int* tok_slot; const int* remain;  // packed form with a cache
  void* cq;                                // [T, q_rank] or null
  void* lat;                               // [T, r + rot] or null
  void* cache;                             // [n_slots, R, r + rot] or null
  int q_rank, r, rot, R;
  float eps;
};

__global__ void __launch_bounds__(128) latent_rope_prepare_kernel(PrepParams p) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int tid = threadIdx.x, dt = p.dt;
  rb::pdl_trigger();
  rb::pdl_wait();
  const int64_t base = t * p.ld;
  int position;
  int64_t crow = -1;
  if (p.pos != nullptr) {
    position = p.pos[t];
    if (p.cache != nullptr && p.tok_slot[t] >= 0 && p.remain[t] < p.R) crow = (int64_t)p.tok_slot[t] * p.R + position % p.R;
  } else {
    const int64_t slot = p.slots ? p.slots[t] : t;
    position = p.lens[slot];
    if (p.cache != nullptr) crow = slot * p.R + position % p.R;
  }
  const int w = p.r + p.rot;
  if (p.q_rank > 0) {
    float ss = 0.f;
    for (int c = tid; c < p.q_rank; c += blockDim.x) { const float v = ld_any(p.proj, dt, base + c); ss += v * v; }
    ss = rb::block_reduce<false>(ss, red);
    const float rs = 1.f / sqrtf(ss / (float)p.q_rank + p.eps);
    for (int c = tid; c < p.q_rank; c += blockDim.x)
      st_any(p.cq, dt, t * p.q_rank + c, ld_any(p.proj, dt, base + c) * rs * ld_any(p.wq, dt, c));
  }
  const int64_t cb = base + p.q_rank;
  float ss = 0.f;
  for (int c = tid; c < p.r; c += blockDim.x) { const float v = ld_any(p.proj, dt, cb + c); ss += v * v; }
  ss = rb::block_reduce<false>(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)p.r + p.eps);
  for (int c = tid; c < p.r; c += blockDim.x) {
    const float v = ld_any(p.proj, dt, cb + c) * rs * ld_any(p.wc, dt, c);
    if (p.lat) st_any(p.lat, dt, t * w + c, v);
    if (crow >= 0) st_any(p.cache, dt, crow * w + c, v);
  }
  const float fp = (float)position;
  for (int i = tid; i < p.rot / 2; i += blockDim.x) {
    float sn, cs;
    sincosf(fp * p.inv_freq[i], &sn, &cs);
    sn *= p.mscale; cs *= p.mscale;
    const float u = ld_any(p.proj, dt, cb + p.r + 2 * i), v = ld_any(p.proj, dt, cb + p.r + 2 * i + 1);
    const float a = u * cs - v * sn, b = v * cs + u * sn;
    if (p.lat) { st_any(p.lat, dt, t * w + p.r + 2 * i, a); st_any(p.lat, dt, t * w + p.r + 2 * i + 1, b); }
    if (crow >= 0) { st_any(p.cache, dt, crow * w + p.r + 2 * i, a); st_any(p.cache, dt, crow * w + p.r + 2 * i + 1, b); }
  }
}

__global__ void __launch_bounds__(256) latent_rope_assemble_kernel(const void* __restrict__ q, int64_t ldq, const void* __restrict__ kn, int64_t ldk,
                                                                    const void* __restrict__ lat, int64_t ldl, int r, const int* __restrict__ pos,
                                                                    const float* __restrict__ inv_freq, float mscale, void* __restrict__ out, int dt,
                                                                    int H, int d, int rot) {
  const int64_t t = blockIdx.x;
  const int dq = d + rot;
  rb::pdl_trigger();
  rb::pdl_wait();
  const float fp = (float)pos[t];
  const int64_t ob = t * (int64_t)(2 * H * dq);
  for (int idx = threadIdx.x; idx < H * dq; idx += blockDim.x) {
    const int h = idx / dq, e = idx % dq;
    if (e < d) {
      st_any(out, dt, ob + idx, ld_any(q, dt, t * ldq + idx));
      st_any(out, dt, ob + H * dq + idx, ld_any(kn, dt, t * ldk + h * d + e));
    } else {
      const int j = e - d, i = j >> 1;
      st_any(out, dt, ob + H * dq + idx, ld_any(lat, dt, t * ldl + r + j));
      if ((j & 1) == 0) {
        float sn, cs;
        sincosf(fp * inv_freq[i], &sn, &cs);
        sn *= mscale; cs *= mscale;
        const float u = ld_any(q, dt, t * ldq + idx), v = ld_any(q, dt, t * ldq + idx + 1);
        st_any(out, dt, ob + idx, u * cs - v * sn);
        st_any(out, dt, ob + idx + 1, v * cs + u * sn);
      }
    }
  }
}

__global__ void __launch_bounds__(128) latent_query_rope_kernel(const void* __restrict__ q, int64_t ldq, int dt, const int* __restrict__ lens,
                                                                 const int* __restrict__ slots, const float* __restrict__ inv_freq, float mscale,
                                                                 float scale, float* __restrict__ qa, int B, int H, int d, int rot, int r) {
  const int b = blockIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  const float fp = (float)lens[slots ? slots[b] : b];
  const int dq = d + rot, w = r + rot;
  for (int idx = threadIdx.x; idx < H * (rot / 2); idx += blockDim.x) {
    const int h = idx / (rot / 2), i = idx % (rot / 2);
    float sn, cs;
    sincosf(fp * inv_freq[i], &sn, &cs);
    sn *= mscale; cs *= mscale;
    const int64_t src = (int64_t)b * ldq + h * dq + d + 2 * i;
    const float u = ld_any(q, dt, src), v = ld_any(q, dt, src + 1);
    float* dst = qa + ((int64_t)h * B + b) * w + r + 2 * i;
    dst[0] = (u * cs - v * sn) * scale;
    dst[1] = (v * cs + u * sn) * scale;
  }
}

__global__ void sigmoid_gate_kernel(void* __restrict__ x, int dtx, const void* __restrict__ g, int64_t ldg, int dtg, int64_t n, int W, int vec4) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  rb::pdl_trigger();
  rb::pdl_wait();
  if (vec4) {                                  // 4 elements per thread (rows and base addresses allow 8- / 16-byte accesses)
    const int64_t i4 = i * 4;
    if (i4 >= n) return;
    const int64_t t = i4 / W;
    const int c = (int)(i4 % W);
    const float4 gv = rb::ld4_any(g, dtg, t * ldg + c), xv = rb::ld4_any(x, dtx, i4);
    rb::st4_any(x, dtx, i4, make_float4(xv.x / (1.f + expf(-gv.x)), xv.y / (1.f + expf(-gv.y)), xv.z / (1.f + expf(-gv.z)), xv.w / (1.f + expf(-gv.w))));
    return;
  }
  if (i >= n) return;
  const int64_t t = i / W;
  const int c = (int)(i % W);
  const float gv = ld_any(g, dtg, t * ldg + c);
  st_any(x, dtx, i, ld_any(x, dtx, i) * (1.f / (1.f + expf(-gv))));
}

}  // namespace

extern "C" int rb_latent_rope_prepare(const void* proj, int64_t ld, int dt, const void* wq, const void* wc, const float* inv_freq, float mscale,
                                      const int* pos, const int* lens, const int* slots, const int* tok_slot, const int* remain, void* cq, void* lat,
                                      void* cache, int64_t T, int q_rank, int r, int rot, int R, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (rot & 1) return -1;
  PrepParams p{proj, ld, dt, wq, wc, inv_freq, mscale, pos, lens, slots, tok_slot, remain, cq, lat, cache, q_rank, r, rot, R, eps};
  return rb::launch_pdl(latent_rope_prepare_kernel, dim3((unsigned)T), dim3(128), 0, s, p) == cudaSuccess ? 0 : 2;
}

extern "C" int rb_latent_rope_assemble(const void* q, int64_t ldq, const void* kn, int64_t ldk, const void* lat, int64_t ldl, int r, const int* pos,
                                       const float* inv_freq, float mscale, void* out, int dt, int64_t T, int H, int d, int rot, cudaStream_t s) {
  if (T == 0) return 0;
  if (rot & 1) return -1;
  return rb::launch_pdl(latent_rope_assemble_kernel, dim3((unsigned)T), dim3(256), 0, s, q, ldq, kn, ldk, lat, ldl, r, pos, inv_freq, mscale, out, dt,
                        H, d, rot) == cudaSuccess ? 0 : 2;
}

extern "C" int rb_latent_query_rope(const void* q, int64_t ldq, int dt, const int* lens, const int* slots, const float* inv_freq, float mscale,
                                    float scale, float* qa, int B, int H, int d, int rot, int r, cudaStream_t s) {
  if (B == 0 || rot == 0) return 0;
  if (rot & 1) return -1;
  return rb::launch_pdl(latent_query_rope_kernel, dim3((unsigned)B), dim3(128), 0, s, q, ldq, dt, lens, slots, inv_freq, mscale, scale, qa, B, H, d, rot,
                        r) == cudaSuccess ? 0 : 2;
}

extern "C" int rb_sigmoid_gate(void* x, int dtx, const void* g, int64_t ldg, int dtg, int64_t T, int W, cudaStream_t s) {
  const int64_t n = T * W;
  if (n == 0) return 0;
  const int vec4 = (W & 3) == 0 && (ldg & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(g) & 15) == 0;
  const int64_t work = vec4 ? n / 4 : n;
  return rb::launch_pdl(sigmoid_gate_kernel, dim3((unsigned)RB_CEIL_DIV(work, (int64_t)256)), dim3(256), 0, s, x, dtx, g, ldg, dtg, n, W, vec4) == cudaSuccess ? 0 : 2;
}
