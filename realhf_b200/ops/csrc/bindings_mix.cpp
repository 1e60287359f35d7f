// torch.ops.realhf_b200.* registrations of the matrix-memory LSTM (mlstm.cu), the rotated latent attention helpers (latent_rope.cu)
// and the query / key head norm and differential combine of window attention (sinkattn.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

using at::Tensor;
using OptT = c10::optional<Tensor>;

#define CHECK_CUDA(x) TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor")
#define CHECK_IN(x) \
  CHECK_CUDA(x);    \
  TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")
#define CHECK_ROWS(x) \
  CHECK_CUDA(x);      \
  TORCH_CHECK((x).dim() == 2 && (x).stride(1) == 1, #x " must be 2-D with unit column stride")

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static inline int dt_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kBFloat16: return 1;
    case at::kHalf: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
}
static inline const int* int_ptr(const OptT& t, int64_t n, const char* what) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kInt && t->numel() >= n, what, ": int32 CUDA tensor expected");
  return t->data_ptr<int>();
}

extern "C" {
int rb_mlstm_scan(const void*, int64_t, int, const void*, float*, float*, const int*, float*, float*, const int*, int, int, int, int, int, int, int, float,
                  float, int, cudaStream_t);
int rb_mlstm_out(const float*, const float*, const void*, int, const void*, int64_t, int, void*, int, int64_t, int, int, float, cudaStream_t);
int rb_latent_rope_prepare(const void*, int64_t, int, const void*, const void*, const float*, float, const int*, const int*, const int*, const int*,
                           const int*, void*, void*, void*, int64_t, int, int, int, int, float, cudaStream_t);
int rb_latent_rope_assemble(const void*, int64_t, const void*, int64_t, const void*, int64_t, int, const int*, const float*, float, void*, int, int64_t,
                            int, int, int, cudaStream_t);
int rb_latent_query_rope(const void*, int64_t, int, const int*, const int*, const float*, float, float, float*, int, int, int, int, int, cudaStream_t);
int rb_sigmoid_gate(void*, int, const void*, int64_t, int, int64_t, int, cudaStream_t);
int rb_softmax_router(const void*, int64_t, int, const void*, int, const void*, int, const void*, int, float*, int64_t*, float*, int64_t, int, int, int,
                      int, int, cudaStream_t);
int rb_moe_combine(const void*, int, const void*, int64_t, int, const int64_t*, const float*, const int64_t*, const void*, int, const float*, void*, int,
                   int64_t, int, int, int, int, cudaStream_t);
int rb_moe_dispatch(const int64_t*, int64_t*, int*, int, int, int, cudaStream_t);
int rb_moe_gather(const void*, int64_t, int, const int64_t*, const float*, void*, int64_t, int, int, cudaStream_t);
int rb_centred_norm(void*, int, const void*, int64_t, const void*, int64_t, int, float, float, const void*, const void*, const void*, int, float, void*,
                    int, int64_t, int, float, cudaStream_t);
int rb_rotate_heads(void*, int64_t, int, const int*, const int*, const int*, const float*, int64_t, int, int, int, int, cudaStream_t);
int rb_decay_prepare(const void*, int64_t, int, float*, const int*, const int*, const int*, const float*, int64_t, int, int, int, int, int, int, float,
                     cudaStream_t);
int rb_decay_scan(const float*, int64_t, const float*, float*, const int*, float*, const int*, int, int, int, int, int, cudaStream_t);
int rb_decay_out(const float*, const void*, int, const void*, int64_t, int, void*, int, int64_t, int, int, float, int, int, cudaStream_t);
int rb_qk_head_norm(void*, int64_t, int, const void*, const void*, int64_t, int, int, int, float, cudaStream_t);
int rb_diff_combine(const void*, int, const float*, void*, int, int64_t, int, int, int, float, float, cudaStream_t);
}

namespace {

// proj [T, ld] = [q (H d) | k (H d) | v (H dv) | output gate (H dv) | x_i (H), x_f (H), padding]; cu absent: decode step (row b =
// sequence b); state [n_slots, H, d, dv + 1] fp32 and m_state [n_slots, H] fp32 or absent.  o [T, H, dv + 1], m_out [T, H] fp32.
void mlstm_scan(const Tensor& proj, const Tensor& gate_bias, Tensor o, Tensor m_out, const OptT& cu, const OptT& state, const OptT& m_state,
                const OptT& slots, int64_t H, int64_t d, int64_t dv, double cap, bool load_state) {
  CHECK_ROWS(proj); CHECK_IN(gate_bias); CHECK_IN(o); CHECK_IN(m_out);
  const int64_t T = proj.size(0);
  const int64_t off_k = H * d, off_v = 2 * H * d, off_if = 2 * H * d + 2 * H * dv;
  TORCH_CHECK(proj.size(1) >= off_if + 2 * H && gate_bias.numel() == 2 * H && gate_bias.scalar_type() == proj.scalar_type());
  TORCH_CHECK(o.scalar_type() == at::kFloat && m_out.scalar_type() == at::kFloat && o.numel() == T * H * (dv + 1) && m_out.numel() == T * H);
  int n_seqs = (int)T;
  const int* cup = nullptr;
  if (cu.has_value()) {
    CHECK_IN((*cu));
    TORCH_CHECK(cu->scalar_type() == at::kInt && cu->numel() >= 1);
    cup = cu->data_ptr<int>();
    n_seqs = (int)cu->numel() - 1;
  }
  float *sp = nullptr, *mp = nullptr;
  if (state.has_value()) {
    CHECK_IN((*state)); CHECK_IN((*m_state));
    TORCH_CHECK(state->scalar_type() == at::kFloat && state->dim() == 4 && state->size(1) == H && state->size(2) == d && state->size(3) == dv + 1);
    TORCH_CHECK(m_state->scalar_type() == at::kFloat && m_state->numel() == state->size(0) * H);
    TORCH_CHECK(slots.has_value() || state->size(0) >= n_seqs);
    sp = state->data_ptr<float>(); mp = m_state->data_ptr<float>();
  }
  TORCH_CHECK(!load_state || sp != nullptr, "load_state needs the state");
  c10::cuda::CUDAGuard g(proj.device());
  const int rc = rb_mlstm_scan(proj.data_ptr(), proj.stride(0), dt_code(proj), gate_bias.data_ptr(), o.data_ptr<float>(), m_out.data_ptr<float>(), cup, sp,
                               mp, int_ptr(slots, n_seqs, "slots"), n_seqs, (int)H, (int)d, (int)dv, (int)off_k, (int)off_v, (int)off_if, (float)cap,
                               (float)(1.0 / std::sqrt((double)d)), load_state ? 1 : 0, cur_stream());
  TORCH_CHECK(rc == 0, "mlstm_scan: unsupported shape (rc ", rc, ")");
}

void mlstm_out(const Tensor& o, const Tensor& m, const Tensor& w, const Tensor& gate, Tensor out, double eps) {
  CHECK_IN(o); CHECK_IN(m); CHECK_IN(w); CHECK_ROWS(gate); CHECK_IN(out);
  TORCH_CHECK(o.dim() == 3 && o.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat);
  const int64_t T = o.size(0), H = o.size(1), dv = o.size(2) - 1;
  TORCH_CHECK(m.numel() == T * H && w.numel() == H * dv && gate.size(0) == T && gate.size(1) >= H * dv && out.numel() == T * H * dv);
  c10::cuda::CUDAGuard g(o.device());
  TORCH_CHECK(rb_mlstm_out(o.data_ptr<float>(), m.data_ptr<float>(), w.data_ptr(), dt_code(w), gate.data_ptr(), gate.stride(0), dt_code(gate),
                           out.data_ptr(), dt_code(out), T, (int)H, (int)dv, (float)eps, cur_stream()) == 0);
}

// pos given: packed form (cache / tok_slot / remain optional); pos absent: step form (position lens[slot], the cache row is written)
void latent_rope_prepare(const Tensor& proj, const OptT& wq, const Tensor& wc, const Tensor& inv_freq, double mscale, const OptT& pos, const OptT& lens,
                         const OptT& slots, const OptT& tok_slot, const OptT& remain, const OptT& cq, const OptT& lat, const OptT& cache, int64_t q_rank,
                         int64_t r, int64_t rot, double eps) {
  CHECK_ROWS(proj); CHECK_IN(wc); CHECK_IN(inv_freq);
  const int64_t T = proj.size(0);
  TORCH_CHECK(proj.size(1) >= q_rank + r + rot && wc.numel() == r && wc.scalar_type() == proj.scalar_type());
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.numel() >= rot / 2 && rot % 2 == 0);
  const void* wqp = nullptr;
  void *cqp = nullptr, *latp = nullptr, *cachep = nullptr;
  if (q_rank > 0) {
    TORCH_CHECK(wq.has_value() && cq.has_value());
    CHECK_IN((*wq)); CHECK_IN((*cq));
    TORCH_CHECK(wq->numel() == q_rank && wq->scalar_type() == proj.scalar_type() && cq->numel() == T * q_rank && cq->scalar_type() == proj.scalar_type());
    wqp = wq->data_ptr(); cqp = cq->data_ptr();
  }
  if (lat.has_value()) {
    CHECK_IN((*lat));
    TORCH_CHECK(lat->numel() == T * (r + rot) && lat->scalar_type() == proj.scalar_type());
    latp = lat->data_ptr();
  }
  int R = 1;
  if (cache.has_value()) {
    CHECK_IN((*cache));
    TORCH_CHECK(cache->dim() == 3 && cache->size(2) == r + rot && cache->scalar_type() == proj.scalar_type());
    R = (int)cache->size(1);
    cachep = cache->data_ptr();
    TORCH_CHECK(pos.has_value() ? (tok_slot.has_value() && remain.has_value()) : (slots.has_value() || cache->size(0) >= T));
  }
  TORCH_CHECK(pos.has_value() || lens.has_value(), "positions: `pos` (packed) or `lens` (step)");
  c10::cuda::CUDAGuard g(proj.device());
  const int rc = rb_latent_rope_prepare(proj.data_ptr(), proj.stride(0), dt_code(proj), wqp, wc.data_ptr(), inv_freq.data_ptr<float>(), (float)mscale,
                                        int_ptr(pos, T, "pos"), pos.has_value() ? nullptr : int_ptr(lens, 1, "lens"),
                                        pos.has_value() ? nullptr : int_ptr(slots, T, "slots"),
                                        cachep && pos.has_value() ? int_ptr(tok_slot, T, "tok_slot") : nullptr,
                                        cachep && pos.has_value() ? int_ptr(remain, T, "remain") : nullptr, cqp, latp, cachep, T, (int)q_rank, (int)r,
                                        (int)rot, R, (float)eps, cur_stream());
  TORCH_CHECK(rc == 0, "latent_rope_prepare: unsupported shape (rc ", rc, ")");
}

void latent_rope_assemble(const Tensor& q, const Tensor& kn, const Tensor& lat, const Tensor& pos, const Tensor& inv_freq, double mscale, Tensor out,
                          int64_t H, int64_t d, int64_t rot, int64_t r) {
  CHECK_ROWS(q); CHECK_ROWS(kn); CHECK_ROWS(lat); CHECK_IN(pos); CHECK_IN(inv_freq); CHECK_IN(out);
  const int64_t T = q.size(0);
  TORCH_CHECK(q.size(1) >= H * (d + rot) && kn.size(1) >= H * d && lat.size(1) >= r + rot && out.numel() == T * 2 * H * (d + rot));
  TORCH_CHECK(kn.scalar_type() == q.scalar_type() && lat.scalar_type() == q.scalar_type() && out.scalar_type() == q.scalar_type());
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.numel() >= rot / 2);
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(rb_latent_rope_assemble(q.data_ptr(), q.stride(0), kn.data_ptr(), kn.stride(0), lat.data_ptr(), lat.stride(0), (int)r,
                                      int_ptr(pos, T, "pos"), inv_freq.data_ptr<float>(), (float)mscale, out.data_ptr(), dt_code(q), T, (int)H, (int)d,
                                      (int)rot, cur_stream()) == 0);
}

// qa [H, B, r + rot] fp32: columns [r, r + rot) <- scale * rotate(q[b, h, d:])
void latent_query_rope(const Tensor& q, const Tensor& lens, const OptT& slots, const Tensor& inv_freq, double mscale, double scale, Tensor qa,
                       int64_t d, int64_t rot) {
  CHECK_ROWS(q); CHECK_IN(lens); CHECK_IN(inv_freq); CHECK_IN(qa);
  TORCH_CHECK(qa.dim() == 3 && qa.scalar_type() == at::kFloat && qa.size(1) == q.size(0) && qa.size(2) > rot);
  const int64_t H = qa.size(0), B = qa.size(1), r = qa.size(2) - rot;
  TORCH_CHECK(q.size(1) >= H * (d + rot) && inv_freq.scalar_type() == at::kFloat && inv_freq.numel() >= rot / 2);
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(rb_latent_query_rope(q.data_ptr(), q.stride(0), dt_code(q), int_ptr(lens, 1, "lens"), int_ptr(slots, B, "slots"),
                                   inv_freq.data_ptr<float>(), (float)mscale, (float)scale, qa.data_ptr<float>(), (int)B, (int)H, (int)d, (int)rot, (int)r,
                                   cur_stream()) == 0);
}

void sigmoid_gate_(Tensor x, const Tensor& gate) {
  CHECK_IN(x); CHECK_ROWS(gate);
  TORCH_CHECK(x.dim() == 2 && gate.size(0) == x.size(0) && gate.size(1) >= x.size(1));
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(rb_sigmoid_gate(x.data_ptr(), dt_code(x), gate.data_ptr(), gate.stride(0), dt_code(gate), x.size(0), (int)x.size(1), cur_stream()) == 0);
}

void qk_head_norm_(Tensor x, const Tensor& wq, const Tensor& wk, int64_t nq, int64_t nk, int64_t d, double eps) {
  CHECK_ROWS(x); CHECK_IN(wq); CHECK_IN(wk);
  TORCH_CHECK(x.size(1) >= (nq + nk) * d && wq.numel() == d && wk.numel() == d && wq.scalar_type() == x.scalar_type() && wk.scalar_type() == x.scalar_type());
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(rb_qk_head_norm(x.data_ptr(), x.stride(0), dt_code(x), wq.data_ptr(), wk.data_ptr(), x.size(0), (int)nq, (int)nk, (int)d, (float)eps,
                              cur_stream()) == 0);
}

void diff_combine(const Tensor& a, const Tensor& lam, Tensor out, int64_t H, int64_t G, int64_t dv, double diff, double eps) {
  CHECK_IN(a); CHECK_IN(lam); CHECK_IN(out);
  TORCH_CHECK(lam.scalar_type() == at::kFloat && lam.numel() == 1 && a.numel() == 2 * out.numel() && out.numel() % (H * dv) == 0 && H % G == 0);
  c10::cuda::CUDAGuard g(a.device());
  TORCH_CHECK(rb_diff_combine(a.data_ptr(), dt_code(a), lam.data_ptr<float>(), out.data_ptr(), dt_code(out), out.numel() / (H * dv), (int)H, (int)G,
                              (int)dv, (float)diff, (float)eps, cur_stream()) == 0);
}

// x [T, K], w [R, K] -> (weights [T, k] fp32, outputs [T, k] int64, gate [T] fp32 or empty): see moe_route.cu
std::vector<Tensor> softmax_router(const Tensor& x, const Tensor& w, const OptT& corr, const OptT& u, int64_t k, bool renorm, bool sigmoid) {
  CHECK_ROWS(x); CHECK_IN(w);
  const int64_t T = x.size(0), K = x.size(1), R = w.size(0);
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && w.size(1) == K && R <= 64 && k >= 1 && k <= 8 && k <= R, "softmax_router: shapes");
  if (corr.has_value()) { CHECK_IN((*corr)); TORCH_CHECK(corr->numel() == R); }
  if (u.has_value()) { CHECK_IN((*u)); TORCH_CHECK(u->numel() == K); }
  c10::cuda::CUDAGuard g(x.device());
  Tensor probs = at::empty({T, k}, x.options().dtype(at::kFloat)), idx = at::empty({T, k}, x.options().dtype(at::kLong));
  Tensor gate = at::empty({u.has_value() ? T : 0}, x.options().dtype(at::kFloat));
  TORCH_CHECK(rb_softmax_router(x.data_ptr(), x.stride(0), dt_code(x), w.data_ptr(), dt_code(w), corr.has_value() ? corr->data_ptr() : nullptr,
                                corr.has_value() ? dt_code(*corr) : 0, u.has_value() ? u->data_ptr() : nullptr, u.has_value() ? dt_code(*u) : 0,
                                probs.data_ptr<float>(), idx.data_ptr<int64_t>(), u.has_value() ? gate.data_ptr<float>() : nullptr, T, (int)K, (int)R,
                                (int)k, renorm ? 1 : 0, sigmoid ? 1 : 0, cur_stream()) == 0);
  return {probs, idx, gate};
}

// out[t] = sum_j probs[t, j] * (idx[t, j] < E ? y[row[t, j]] : x[t]) + gate[t] * y_shared[t]   (unit: probs read as 1; no gate: 1)
void moe_combine(const Tensor& y, const Tensor& x, const Tensor& row, const Tensor& probs, const Tensor& idx, const OptT& ysh, const OptT& gate,
                 Tensor out, int64_t E, bool unit) {
  CHECK_IN(y); CHECK_ROWS(x); CHECK_IN(row); CHECK_IN(probs); CHECK_IN(idx); CHECK_IN(out);
  const int64_t T = x.size(0), H = x.size(1), k = probs.size(1);
  TORCH_CHECK(y.dim() == 2 && y.size(1) == H && out.size(0) == T && out.size(1) == H && probs.size(0) == T && idx.numel() == T * k && row.numel() == T * k);
  TORCH_CHECK(row.scalar_type() == at::kLong && idx.scalar_type() == at::kLong && probs.scalar_type() == at::kFloat && k <= 8);
  TORCH_CHECK(ysh.has_value() || !gate.has_value());
  if (ysh.has_value()) {
    CHECK_IN((*ysh));
    TORCH_CHECK(ysh->size(0) == T && ysh->size(1) == H);
  }
  if (gate.has_value()) {
    CHECK_IN((*gate));
    TORCH_CHECK(gate->numel() == T && gate->scalar_type() == at::kFloat);
  }
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(rb_moe_combine(y.data_ptr(), dt_code(y), x.data_ptr(), x.stride(0), dt_code(x), row.data_ptr<int64_t>(), probs.data_ptr<float>(),
                             idx.data_ptr<int64_t>(), ysh.has_value() ? ysh->data_ptr() : nullptr, ysh.has_value() ? dt_code(*ysh) : 0,
                             gate.has_value() ? gate->data_ptr<float>() : nullptr, out.data_ptr(), dt_code(out), T, (int)H, (int)k, (int)E,
                             unit ? 1 : 0, cur_stream()) == 0);
}

// idx [T, k] int64 (router outputs, E real experts of R) -> (row [T k] int64: place of each assignment in the order sorted by expert,
// offsets [E + 1] int32: first row of each real expert); T k <= 1024
std::vector<Tensor> moe_dispatch(const Tensor& idx, int64_t E, int64_t R) {
  CHECK_IN(idx);
  const int64_t N = idx.numel();
  TORCH_CHECK(idx.scalar_type() == at::kLong && N >= 1 && N <= 1024 && R <= 64 && E <= R, "moe_dispatch: shapes");
  c10::cuda::CUDAGuard g(idx.device());
  Tensor row = at::empty({N}, idx.options()), offsets = at::empty({E + 1}, idx.options().dtype(at::kInt));
  TORCH_CHECK(rb_moe_dispatch(idx.data_ptr<int64_t>(), row.data_ptr<int64_t>(), offsets.data_ptr<int>(), (int)N, (int)E, (int)R, cur_stream()) == 0);
  return {row, offsets};
}

// x [T, H], row [T k] -> xs [T k, H] with xs[row[i]] = x[i / k] (times scale[i], fp32 [T k], when given)
Tensor moe_gather(const Tensor& x, const Tensor& row, int64_t k, const OptT& scale) {
  CHECK_ROWS(x); CHECK_IN(row);
  TORCH_CHECK(row.scalar_type() == at::kLong && row.numel() == x.size(0) * k);
  if (scale.has_value()) { CHECK_IN((*scale)); TORCH_CHECK(scale->scalar_type() == at::kFloat && scale->numel() == row.numel()); }
  c10::cuda::CUDAGuard g(x.device());
  Tensor xs = at::empty({row.numel(), x.size(1)}, x.options());
  TORCH_CHECK(rb_moe_gather(x.data_ptr(), x.stride(0), dt_code(x), row.data_ptr<int64_t>(), scale.has_value() ? scale->data_ptr<float>() : nullptr,
                            xs.data_ptr(), row.numel(), (int)x.size(1), (int)k, cur_stream()) == 0);
  return xs;
}

// "layer" stacks (centred_norm.cu): res += mult * scale * LN(a y + b y2) * w_post, out = LN(res or the branch) * w_next
void centred_norm(const OptT& res, const Tensor& y, const OptT& y2, double a, double b, const OptT& w_post, const OptT& scale, double mult,
                  const OptT& w_next, const OptT& out, double eps) {
  CHECK_ROWS(y);
  const int64_t T = y.size(0), W = y.size(1);
  const Tensor* wv = w_post.has_value() ? &*w_post : (w_next.has_value() ? &*w_next : nullptr);
  TORCH_CHECK(wv != nullptr && w_next.has_value() == out.has_value() && (res.has_value() || out.has_value()), "centred_norm: arguments");
  for (const OptT* o : {&w_post, &scale, &w_next})
    if (o->has_value()) { CHECK_IN((**o)); TORCH_CHECK((*o)->numel() == W && (*o)->scalar_type() == wv->scalar_type()); }
  if (res.has_value()) { CHECK_IN((*res)); TORCH_CHECK(res->numel() == T * W && w_post.has_value()); }
  if (y2.has_value()) { CHECK_ROWS((*y2)); TORCH_CHECK(y2->size(0) == T && y2->size(1) == W && y2->scalar_type() == y.scalar_type()); }
  if (out.has_value()) { CHECK_IN((*out)); TORCH_CHECK(out->numel() == T * W); }
  c10::cuda::CUDAGuard g(y.device());
  TORCH_CHECK(rb_centred_norm(res.has_value() ? res->data_ptr() : nullptr, res.has_value() ? dt_code(*res) : 0, y.data_ptr(), y.stride(0),
                              y2.has_value() ? y2->data_ptr() : nullptr, y2.has_value() ? y2->stride(0) : 0, dt_code(y), (float)a, (float)b,
                              w_post.has_value() ? w_post->data_ptr() : nullptr, scale.has_value() ? scale->data_ptr() : nullptr,
                              w_next.has_value() ? w_next->data_ptr() : nullptr, dt_code(*wv), (float)mult,
                              out.has_value() ? out->data_ptr() : nullptr, out.has_value() ? dt_code(*out) : 0, T, (int)W, (float)eps,
                              cur_stream()) == 0);
}

// in place: the n_h heads of size d at the start of every row of x turn by the row's position (decay.cu)
void rotate_heads_(Tensor x, const OptT& pos, const OptT& lens, const OptT& slots, const Tensor& inv_freq, int64_t n_h, int64_t d, int64_t dims,
                   bool interleaved) {
  CHECK_ROWS(x); CHECK_IN(inv_freq);
  const int64_t T = x.size(0);
  TORCH_CHECK(x.size(1) >= n_h * d && inv_freq.scalar_type() == at::kFloat && inv_freq.numel() >= dims / 2 && (pos.has_value() || lens.has_value()));
  c10::cuda::CUDAGuard g(x.device());
  TORCH_CHECK(rb_rotate_heads(x.data_ptr(), x.stride(0), dt_code(x), int_ptr(pos, T, "pos"), int_ptr(lens, 1, "lens"), int_ptr(slots, T, "slots"),
                              inv_freq.data_ptr<float>(), T, (int)n_h, (int)d, (int)dims, interleaved ? 1 : 0, cur_stream()) == 0);
}

// proj [T, ld] = [q (H d) | k (H d) | v (H dv) | ..] -> u [T, 2 H d + H dv] fp32 (decay.cu)
void decay_prepare(const Tensor& proj, Tensor u, const OptT& pos, const OptT& lens, const OptT& slots, const OptT& inv_freq, int64_t H, int64_t d,
                   int64_t dv, int64_t dims, bool interleaved, bool silu, double k_scale) {
  CHECK_ROWS(proj); CHECK_IN(u);
  const int64_t T = proj.size(0), n = 2 * H * d + H * dv;
  TORCH_CHECK(proj.size(1) >= n && u.scalar_type() == at::kFloat && u.numel() == T * n);
  const float* fp = nullptr;
  if (dims > 0) {
    TORCH_CHECK(inv_freq.has_value() && (pos.has_value() || lens.has_value()));
    CHECK_IN((*inv_freq));
    TORCH_CHECK(inv_freq->scalar_type() == at::kFloat && inv_freq->numel() >= dims / 2);
    fp = inv_freq->data_ptr<float>();
  }
  c10::cuda::CUDAGuard g(proj.device());
  TORCH_CHECK(rb_decay_prepare(proj.data_ptr(), proj.stride(0), dt_code(proj), u.data_ptr<float>(), int_ptr(pos, T, "pos"), int_ptr(lens, 1, "lens"),
                               int_ptr(slots, T, "slots"), fp, T, (int)H, (int)d, (int)dv, (int)dims, interleaved ? 1 : 0, silu ? 1 : 0,
                               (float)k_scale, cur_stream()) == 0);
}

// u [T, 2 H d + H dv] fp32; cu absent: decode step (row b = sequence b); state [n_slots, H, d, dv] fp32 or absent.  o [T, H, dv] fp32.
void decay_scan(const Tensor& u, const Tensor& decay, Tensor o, const OptT& cu, const OptT& state, const OptT& slots, int64_t H, int64_t d,
                int64_t dv, bool load_state) {
  CHECK_IN(u); CHECK_IN(decay); CHECK_IN(o);
  const int64_t T = u.size(0);
  TORCH_CHECK(u.scalar_type() == at::kFloat && u.dim() == 2 && u.size(1) == 2 * H * d + H * dv && decay.scalar_type() == at::kFloat &&
              decay.numel() == H && o.scalar_type() == at::kFloat && o.numel() == T * H * dv);
  int n_seqs = (int)T;
  const int* cup = nullptr;
  if (cu.has_value()) {
    CHECK_IN((*cu));
    TORCH_CHECK(cu->scalar_type() == at::kInt && cu->numel() >= 1);
    cup = cu->data_ptr<int>();
    n_seqs = (int)cu->numel() - 1;
  }
  float* sp = nullptr;
  if (state.has_value()) {
    CHECK_IN((*state));
    TORCH_CHECK(state->scalar_type() == at::kFloat && state->dim() == 4 && state->size(1) == H && state->size(2) == d && state->size(3) == dv);
    sp = state->data_ptr<float>();
  }
  TORCH_CHECK(sp != nullptr || !load_state, "decay_scan: load_state needs a state");
  c10::cuda::CUDAGuard g(u.device());
  TORCH_CHECK(rb_decay_scan(u.data_ptr<float>(), u.stride(0), decay.data_ptr<float>(), o.data_ptr<float>(), cup, sp, int_ptr(slots, n_seqs, "slots"),
                            n_seqs, (int)H, (int)d, (int)dv, load_state ? 1 : 0, cur_stream()) == 0);
}

// o [T, H, dv] fp32 -> out [T, H dv]: per-head RMS norm, or one over all heads times w; times silu / sigmoid of gate [T, >= H dv]
void decay_out(const Tensor& o, const OptT& w, const Tensor& gate, Tensor out, double eps, bool full, bool silu) {
  CHECK_IN(o); CHECK_ROWS(gate); CHECK_IN(out);
  TORCH_CHECK(o.dim() == 3 && o.scalar_type() == at::kFloat);
  const int64_t T = o.size(0), H = o.size(1), dv = o.size(2);
  TORCH_CHECK(gate.size(0) == T && gate.size(1) >= H * dv && out.numel() == T * H * dv && (!full || w.has_value()));
  if (w.has_value()) { CHECK_IN((*w)); TORCH_CHECK(w->numel() == H * dv); }
  c10::cuda::CUDAGuard g(o.device());
  TORCH_CHECK(rb_decay_out(o.data_ptr<float>(), w.has_value() ? w->data_ptr() : nullptr, w.has_value() ? dt_code(*w) : 0, gate.data_ptr(),
                           gate.stride(0), dt_code(gate), out.data_ptr(), dt_code(out), T, (int)H, (int)dv, (float)eps, full ? 1 : 0, silu ? 1 : 0,
                           cur_stream()) == 0);
}

}  // namespace

void register_mix_ops(torch::Library& m) {
  m.def("mlstm_scan(Tensor proj, Tensor gate_bias, Tensor(a!) o, Tensor(b!) m_out, Tensor? cu, Tensor(c!)? state, Tensor(d!)? m_state, Tensor? slots, int H, int d, int dv, float cap, bool load_state) -> ()", &mlstm_scan);
  m.def("mlstm_out(Tensor o, Tensor m, Tensor w, Tensor gate, Tensor(a!) out, float eps) -> ()", &mlstm_out);
  m.def("latent_rope_prepare(Tensor proj, Tensor? wq, Tensor wc, Tensor inv_freq, float mscale, Tensor? pos, Tensor? lens, Tensor? slots, Tensor? tok_slot, Tensor? remain, Tensor(a!)? cq, Tensor(b!)? lat, Tensor(c!)? cache, int q_rank, int r, int rot, float eps) -> ()", &latent_rope_prepare);
  m.def("latent_rope_assemble(Tensor q, Tensor kn, Tensor lat, Tensor pos, Tensor inv_freq, float mscale, Tensor(a!) out, int H, int d, int rot, int r) -> ()", &latent_rope_assemble);
  m.def("latent_query_rope(Tensor q, Tensor lens, Tensor? slots, Tensor inv_freq, float mscale, float scale, Tensor(a!) qa, int d, int rot) -> ()", &latent_query_rope);
  m.def("sigmoid_gate_(Tensor(a!) x, Tensor gate) -> ()", &sigmoid_gate_);
  m.def("moe_dispatch(Tensor idx, int E, int R) -> Tensor[]", &moe_dispatch);
  m.def("moe_gather(Tensor x, Tensor row, int k, Tensor? scale=None) -> Tensor", &moe_gather);
  m.def("softmax_router(Tensor x, Tensor w, Tensor? corr, Tensor? u, int k, bool renorm, bool sigmoid=False) -> Tensor[]", &softmax_router);
  m.def("moe_combine(Tensor y, Tensor x, Tensor row, Tensor probs, Tensor idx, Tensor? y_shared, Tensor? gate, Tensor(a!) out, int E, bool unit=False) -> ()", &moe_combine);
  m.def("centred_norm(Tensor(a!)? res, Tensor y, Tensor? y2, float a, float b, Tensor? w_post, Tensor? scale, float mult, Tensor? w_next, Tensor(b!)? out, float eps) -> ()", &centred_norm);
  m.def("rotate_heads_(Tensor(a!) x, Tensor? pos, Tensor? lens, Tensor? slots, Tensor inv_freq, int n_h, int d, int dims, bool interleaved) -> ()", &rotate_heads_);
  m.def("decay_prepare(Tensor proj, Tensor(a!) u, Tensor? pos, Tensor? lens, Tensor? slots, Tensor? inv_freq, int H, int d, int dv, int dims, bool interleaved, bool silu, float k_scale) -> ()", &decay_prepare);
  m.def("decay_scan(Tensor u, Tensor decay, Tensor(a!) o, Tensor? cu, Tensor(b!)? state, Tensor? slots, int H, int d, int dv, bool load_state) -> ()", &decay_scan);
  m.def("decay_out(Tensor o, Tensor? w, Tensor gate, Tensor(a!) out, float eps, bool full, bool silu) -> ()", &decay_out);
  m.def("qk_head_norm_(Tensor(a!) x, Tensor wq, Tensor wk, int nq, int nk, int d, float eps) -> ()", &qk_head_norm_);
  m.def("diff_combine(Tensor a, Tensor lam, Tensor(a!) out, int H, int G, int dv, float diff, float eps) -> ()", &diff_combine);
}
