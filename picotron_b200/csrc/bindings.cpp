// Python bindings of the sm_100a kernels (module picotron_b200._C).
// This file contains no device code: it validates tensors, allocates outputs through the PyTorch
// caching allocator and calls the C launch API of the .cu files on the current CUDA stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

using torch::Tensor;

extern "C" {
int pt_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                 long long ldd, int a_mn, int b_mn, int out_mode, int num_sms, cudaStream_t stream);
void pt_gemm_set_pair(int on);
int pt_gemm_get_pair();
int pt_gemm_bf16_fused(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd,
                       int epi, void* H, long long ldh, int inter, const float* cosT, const float* sinT, int seq, int rot_heads,
                       int head_dim, void* status, cudaStream_t stream);
int pt_gemm_bf16_ce(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb, long long ldd,
                    const long long* targets, long long vocab_start, void* part, float* tgt, void* status, cudaStream_t stream);
int pt_ce_combine(const void* part, float* rowmax, float* sumexp, long long T, int tiles, cudaStream_t st);
void* pt_status_word();
void pt_attention_set_profile(unsigned long long* counters);
void pt_gemm_set_group_m(int g);
int pt_gemm_get_group_m();
void pt_gemm_set_tma_epilogue(int on);
int pt_gemm_get_tma_epilogue();
unsigned int pt_kernel_status_fetch_and_clear();
unsigned long long pt_launch_count();
void pt_count_launches(int n);
int pt_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* x_new, void* y, float* rstd, int T, int H,
                   float eps, cudaStream_t st);
int pt_rmsnorm_bwd_partial_rows(int T, int num_sms);
int pt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                   float* dw, float* partial, int T, int H, int num_sms, cudaStream_t st);
int pt_rmsnorm_bwd_acc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                       float* dw_acc, int T, int H, int num_sms, cudaStream_t st);
int pt_rope(void* qkv, const float* cosT, const float* sinT, long long T, int n_rot, int d, int S,
            long long row_stride, int inverse, cudaStream_t st);
int pt_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t st);
int pt_swiglu_bwd(const void* gu, const void* da, void* dgu, long long T, int I, cudaStream_t st);
int pt_embedding_fwd(const long long* ids, const void* w, void* out, long long T, int H, long long rows,
                     long long vocab_start, cudaStream_t st);
int pt_embedding_bwd(const long long* ids, const void* dy, float* dw, long long T, int H, long long rows,
                     long long vocab_start, cudaStream_t st);
int pt_ce_stats(const void* logits, const long long* targets, float* rowmax, float* sumexp, float* tgt, long long T,
                int V, long long ld, long long vocab_start, cudaStream_t st);
int pt_ce_grad(void* logits, const long long* targets, const float* lse, long long T, int V, long long ld, float scale,
               long long vocab_start, cudaStream_t st);
int pt_accumulate(float* acc, const void* g, long long n, int g_is_f32, cudaStream_t st);
int pt_add(const void* a, const void* b, void* out, long long n, cudaStream_t st);
int pt_adamw_multi(void** params, const float** grads, float** ms, float** vs, float** masters,
                   const long long* numels, int count, int param_is_bf16, int step, float lr, float beta1, float beta2,
                   float eps, float wd, cudaStream_t st);
int pt_merge_attention(float* out, float* lse, const void* bo, const float* bl, int B, int S, int h, int d,
                       cudaStream_t st);
int pt_allreduce_symm(void* const* buf_ptrs, void* const* flag_ptrs, void* mc_ptr, long long offset_elems, long long n,
                      int is_bf16, float scale, int rank, int world, int num_blocks, long long staging_off_bytes, cudaStream_t st);
void pt_set_wait_limit_ns(unsigned long long ns);
int pt_pdl_enabled();
void pt_set_pdl(int on);
unsigned long long pt_get_wait_limit_ns();
int pt_gemm_allreduce_bf16(const void* A, const void* B, void* const* buf_ptrs, void* const* flag_ptrs, void* mc_ptr,
                           long long d_offset,
                           int M, int N, int K, long long lda, long long ldb, long long ldd, int a_mn, int b_mn, int rank,
                           int world, int clusters_cap, cudaStream_t stream);
int pt_symm_barrier(void* const* flag_ptrs, int rank, int world, cudaStream_t st);
int pt_ce_stats_combine_peers(void* const* buf_ptrs, long long offset_bytes, int world, long long n, float* lse, float* tgt,
                              cudaStream_t st);
int pt_embedding_gather_peers(const long long* ids, void* const* shard_ptrs, int world, long long rows_per_rank, long long T, int H,
                              void* out, cudaStream_t st);
int pt_gather_peer(void* dst, const void* const* src_ptrs, int n_src, long long bytes_each, cudaStream_t st);
int pt_reduce_dkv_symm(void* const* buf_ptrs, long long offset_elems, int me, int world, long long tokens, int width,
                       void* dk, void* dv, long long dk_row, long long dv_row, cudaStream_t st);
int pt_attention_fwd_segs(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, int n_segs, void* o,
                          float* lse, int B, int Sq, int Sk, int hq, int hkv, int d, long long q_row, long long k_row,
                          long long v_row, int causal, float scale, cudaStream_t st);
int pt_attention_bwd_segs(const void* dout, const void* q, const void* const* k_ptrs, const void* const* v_ptrs, int n_segs,
                          const void* o, const float* lse, const float* delta_in, float* delta_ws, float* dq_ws, void* dq,
                          void* dk, void* dv, int out_f32, long long seg_stride, int B, int Sq, int Sk, int hq, int hkv,
                          int d, long long q_row, long long k_row, long long v_row, long long dq_row, long long dk_row,
                          long long dv_row, int causal, float scale, cudaStream_t st);
int pt_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk, int hq,
                     int hkv, int d, long long q_row, long long k_row, long long v_row, int causal, float scale,
                     cudaStream_t st);
int pt_attention_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse,
                     const float* delta_in, float* delta_ws, float* dq_ws, void* dq, void* dk, void* dv, int B, int Sq,
                     int Sk, int hq, int hkv, int d, long long q_row, long long k_row, long long v_row,
                     long long dq_row, long long dk_row, long long dv_row, int causal, float scale, cudaStream_t st);
int pt_attention_bwd_rope(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse,
                          const float* delta_in, float* delta_ws, float* dq_ws, void* dq, void* dk, void* dv, int B, int Sq,
                          int Sk, int hq, int hkv, int d, long long q_row, long long k_row, long long v_row, long long dq_row,
                          long long dk_row, long long dv_row, int causal, float scale, const float* cosT, const float* sinT,
                          int rope_seq, cudaStream_t st);
}

namespace {

inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline int num_sms() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }

#define PT_CHECK_RC(rc, what) TORCH_CHECK((rc) == 0, what, " failed with code ", (rc))
#define PT_CHECK_BF16(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kBFloat16, #t " must be a CUDA bf16 tensor")
#define PT_CHECK_F32(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kFloat, #t " must be a CUDA fp32 tensor")

// rows x cols view of a 2-D tensor whose rows are contiguous; returns the row stride in elements
inline long long row_stride_2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() == 2 && (t.size(1) == 1 || t.stride(1) == 1), name, " must be 2-D with contiguous rows");
  return t.size(0) == 1 ? t.size(1) : t.stride(0);
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  PT_CHECK_BF16(x); PT_CHECK_BF16(w);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && w.is_contiguous() && w.numel() == x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  auto rstd = torch::empty({x.size(0)}, x.options().dtype(at::kFloat));
  PT_CHECK_RC(pt_rmsnorm_fwd(x.data_ptr(), nullptr, w.data_ptr(), nullptr, y.data_ptr(), rstd.data_ptr<float>(),
                             (int)x.size(0), (int)x.size(1), (float)eps, stream()), "rmsnorm_fwd");
  return {y, rstd};
}

std::vector<Tensor> add_rmsnorm_fwd(const Tensor& x, const Tensor& delta, const Tensor& w, double eps) {
  PT_CHECK_BF16(x); PT_CHECK_BF16(delta); PT_CHECK_BF16(w);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && delta.is_contiguous() && delta.sizes() == x.sizes() &&
              w.numel() == x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  auto x_new = torch::empty_like(x);
  auto y = torch::empty_like(x);
  auto rstd = torch::empty({x.size(0)}, x.options().dtype(at::kFloat));
  PT_CHECK_RC(pt_rmsnorm_fwd(x.data_ptr(), delta.data_ptr(), w.data_ptr(), x_new.data_ptr(), y.data_ptr(),
                             rstd.data_ptr<float>(), (int)x.size(0), (int)x.size(1), (float)eps, stream()),
              "add_rmsnorm_fwd");
  return {x_new, y, rstd};
}

// Returns {dx, dw}. With `dw_acc` (fp32 [H]) the weight gradient is ADDED to it and returned as the second element.
std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd,
                                const c10::optional<Tensor>& dres, const c10::optional<Tensor>& dw_acc) {
  PT_CHECK_BF16(dy); PT_CHECK_BF16(x); PT_CHECK_BF16(w); PT_CHECK_F32(rstd);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && dy.is_contiguous() && dy.sizes() == x.sizes());
  if (dres.has_value()) { PT_CHECK_BF16(*dres); TORCH_CHECK(dres->is_contiguous() && dres->sizes() == x.sizes()); }
  c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), H = (int)x.size(1);
  if (dw_acc.has_value()) {
    PT_CHECK_F32(*dw_acc);
    TORCH_CHECK(dw_acc->is_contiguous() && dw_acc->numel() == H, "rmsnorm_bwd: dw_acc must be a contiguous fp32 [H] tensor");
  }
  auto dx = torch::empty_like(x);
  // one kernel that adds dw with vector reductions (shapes it covers), else partials + a second kernel
  Tensor dw = dw_acc.has_value() ? *dw_acc : torch::zeros({H}, x.options().dtype(at::kFloat));
  const int rc = pt_rmsnorm_bwd_acc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                                    dres.has_value() ? dres->data_ptr() : nullptr, dx.data_ptr(), dw.data_ptr<float>(), T, H,
                                    num_sms(), stream());
  if (rc == 0) return {dx, dw};
  TORCH_CHECK(rc == 1, "rmsnorm_bwd failed with code ", rc);
  auto dw_new = torch::empty({H}, x.options().dtype(at::kFloat));
  auto partial = torch::empty({pt_rmsnorm_bwd_partial_rows(T, num_sms()), H}, x.options().dtype(at::kFloat));
  PT_CHECK_RC(pt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                             dres.has_value() ? dres->data_ptr() : nullptr, dx.data_ptr(), dw_new.data_ptr<float>(),
                             partial.data_ptr<float>(), T, H, num_sms(), stream()), "rmsnorm_bwd");
  if (dw_acc.has_value()) {
    dw.add_(dw_new);
    return {dx, dw};
  }
  return {dx, dw_new};
}

void rope_(Tensor& qkv, const Tensor& cosT, const Tensor& sinT, int64_t n_rot, int64_t d, int64_t S, bool inverse) {
  PT_CHECK_BF16(qkv); PT_CHECK_F32(cosT); PT_CHECK_F32(sinT);
  TORCH_CHECK(cosT.is_contiguous() && sinT.is_contiguous() && cosT.size(0) >= S && cosT.size(1) == d / 2);
  const long long rs = row_stride_2d(qkv, "qkv");
  TORCH_CHECK(n_rot * d <= qkv.size(1));
  c10::cuda::CUDAGuard guard(qkv.device());
  PT_CHECK_RC(pt_rope(qkv.data_ptr(), cosT.data_ptr<float>(), sinT.data_ptr<float>(), qkv.size(0), (int)n_rot, (int)d,
                      (int)S, rs, inverse ? 1 : 0, stream()), "rope");
}

Tensor swiglu_fwd(const Tensor& gu) {
  PT_CHECK_BF16(gu);
  TORCH_CHECK(gu.dim() == 2 && gu.is_contiguous() && gu.size(1) % 2 == 0);
  c10::cuda::CUDAGuard guard(gu.device());
  auto out = torch::empty({gu.size(0), gu.size(1) / 2}, gu.options());
  PT_CHECK_RC(pt_swiglu_fwd(gu.data_ptr(), out.data_ptr(), gu.size(0), (int)(gu.size(1) / 2), stream()), "swiglu_fwd");
  return out;
}

Tensor swiglu_bwd(const Tensor& gu, const Tensor& da) {
  PT_CHECK_BF16(gu); PT_CHECK_BF16(da);
  TORCH_CHECK(gu.dim() == 2 && gu.is_contiguous() && da.is_contiguous() && da.size(0) == gu.size(0) &&
              da.size(1) * 2 == gu.size(1));
  c10::cuda::CUDAGuard guard(gu.device());
  auto dgu = torch::empty_like(gu);
  PT_CHECK_RC(pt_swiglu_bwd(gu.data_ptr(), da.data_ptr(), dgu.data_ptr(), gu.size(0), (int)da.size(1), stream()),
              "swiglu_bwd");
  return dgu;
}

// gu[T, 2I] = x w_gu^T and h[T, I] = silu(gate) * up from ONE GEMM (SwiGLU epilogue). Returns {} when the fused kernel does
// not cover the case (CTA pairs or the TMA epilogue unavailable, I % 128 != 0): the caller then runs GEMM + activation kernel.
std::vector<Tensor> gemm_swiglu(const Tensor& x, const Tensor& w_gu) {
  PT_CHECK_BF16(x); PT_CHECK_BF16(w_gu);
  const long long lda = row_stride_2d(x, "x"), ldb = row_stride_2d(w_gu, "w_gu");
  const int64_t M = x.size(0), K = x.size(1), N2 = w_gu.size(0);
  TORCH_CHECK(w_gu.size(1) == K && N2 % 2 == 0, "gemm_swiglu: shape mismatch");
  if (!pt_gemm_get_pair() || (N2 / 2) % 128 != 0) return {};
  c10::cuda::CUDAGuard guard(x.device());
  auto gu = torch::empty({M, N2}, x.options());
  auto h = torch::empty({M, N2 / 2}, x.options());
  const int rc = pt_gemm_bf16_fused(x.data_ptr(), w_gu.data_ptr(), gu.data_ptr(), (int)M, (int)N2, (int)K, lda, ldb, N2, 1,
                                    h.data_ptr(), N2 / 2, (int)(N2 / 2), nullptr, nullptr, 0, 0, 0, pt_status_word(), stream());
  if (rc == 1 || rc == -5) return {};
  TORCH_CHECK(rc == 0, "gemm_swiglu failed with code ", rc);
  return {gu, h};
}

// qkv[T, N] = x w^T with RoPE applied to the first `n_rot` heads in the GEMM epilogue. Returns an undefined tensor when
// the fused kernel does not cover the case.
Tensor gemm_rope(const Tensor& x, const Tensor& w, const Tensor& cosT, const Tensor& sinT, int64_t n_rot, int64_t d, int64_t S) {
  PT_CHECK_BF16(x); PT_CHECK_BF16(w); PT_CHECK_F32(cosT); PT_CHECK_F32(sinT);
  const long long lda = row_stride_2d(x, "x"), ldb = row_stride_2d(w, "w");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "gemm_rope: shape mismatch");
  TORCH_CHECK(cosT.is_contiguous() && sinT.is_contiguous() && cosT.size(0) >= S && cosT.size(1) == d / 2 && sinT.sizes() == cosT.sizes());
  if (!pt_gemm_get_pair() || N % 8 != 0) return Tensor();
  c10::cuda::CUDAGuard guard(x.device());
  auto qkv = torch::empty({M, N}, x.options());
  const int rc = pt_gemm_bf16_fused(x.data_ptr(), w.data_ptr(), qkv.data_ptr(), (int)M, (int)N, (int)K, lda, ldb, N, 2, nullptr, 0,
                                    0, cosT.data_ptr<float>(), sinT.data_ptr<float>(), (int)S, (int)n_rot, (int)d,
                                    pt_status_word(), stream());
  if (rc == 1 || rc == -5) return Tensor();
  TORCH_CHECK(rc == 0, "gemm_rope failed with code ", rc);
  return qkv;
}

// y[T, N] = x w^T + res (res: bf16 [T, N], the residual stream) from one GEMM whose epilogue fetches the residual tile with
// TMA and adds it before the single rounding to bf16. Returns an undefined tensor when the fused kernel does not cover the case.
Tensor gemm_add(const Tensor& x, const Tensor& w, const Tensor& res) {
  PT_CHECK_BF16(x); PT_CHECK_BF16(w); PT_CHECK_BF16(res);
  const long long lda = row_stride_2d(x, "x"), ldb = row_stride_2d(w, "w"), ldh = row_stride_2d(res, "res");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && res.size(0) == M && res.size(1) == N, "gemm_add: shape mismatch");
  if (!pt_gemm_get_pair() || N % 8 != 0) return Tensor();
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({M, N}, x.options());
  const int rc = pt_gemm_bf16_fused(x.data_ptr(), w.data_ptr(), y.data_ptr(), (int)M, (int)N, (int)K, lda, ldb, N, 4,
                                    res.data_ptr(), ldh, 0, nullptr, nullptr, 0, 0, 0, pt_status_word(), stream());
  if (rc == 1 || rc == -5) return Tensor();
  TORCH_CHECK(rc == 0, "gemm_add failed with code ", rc);
  return y;
}

// dgu[T, 2I] = SwiGLU backward of (dy w) against the packed pre-activations gu[T, 2I], all in the dgrad GEMM's epilogue
// (dy: [T, H], w: the down-projection weight [H, I]). Returns an undefined tensor when the fused kernel does not cover the case.
Tensor gemm_dgrad_swiglu_bwd(const Tensor& dy, const Tensor& w, const Tensor& gu) {
  PT_CHECK_BF16(dy); PT_CHECK_BF16(w); PT_CHECK_BF16(gu);
  const long long lda = row_stride_2d(dy, "dy"), ldb = row_stride_2d(w, "w"), ldh = row_stride_2d(gu, "gu");
  const int64_t M = dy.size(0), K = dy.size(1), I = w.size(1);
  TORCH_CHECK(w.size(0) == K && gu.size(0) == M && gu.size(1) == 2 * I, "gemm_dgrad_swiglu_bwd: shape mismatch");
  if (!pt_gemm_get_pair() || I % 64 != 0) return Tensor();
  c10::cuda::CUDAGuard guard(dy.device());
  auto dgu = torch::empty({M, 2 * I}, dy.options());
  const int rc = pt_gemm_bf16_fused(dy.data_ptr(), w.data_ptr(), dgu.data_ptr(), (int)M, (int)I, (int)K, lda, ldb, 2 * I, 5,
                                    gu.data_ptr(), ldh, (int)I, nullptr, nullptr, 0, 0, 0, pt_status_word(), stream());
  if (rc == 1 || rc == -5) return Tensor();
  TORCH_CHECK(rc == 0, "gemm_dgrad_swiglu_bwd failed with code ", rc);
  return dgu;
}

// D = op(a) op(b); see pt_gemm_bf16. trans_a: a is [K,M]; trans_b: b is [K,N] (else [N,K]).
Tensor gemm(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b, const c10::optional<Tensor>& out,
            bool accumulate) {
  PT_CHECK_BF16(a); PT_CHECK_BF16(b);
  const long long lda = row_stride_2d(a, "a"), ldb = row_stride_2d(b, "b");
  const int64_t M = trans_a ? a.size(1) : a.size(0), K = trans_a ? a.size(0) : a.size(1);
  const int64_t N = trans_b ? b.size(1) : b.size(0), Kb = trans_b ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: reduction dims differ (", K, " vs ", Kb, ")");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor d;
  int mode;
  if (out.has_value()) {
    d = *out;
    TORCH_CHECK(d.is_cuda() && d.dim() == 2 && d.size(0) == M && d.size(1) == N, "gemm: bad out shape");
    if (d.scalar_type() == at::kFloat) mode = accumulate ? 1 : 2;
    else { TORCH_CHECK(d.scalar_type() == at::kBFloat16 && !accumulate, "gemm: accumulate needs an fp32 out"); mode = 0; }
  } else {
    TORCH_CHECK(!accumulate, "gemm: accumulate needs out");
    d = torch::empty({M, N}, a.options());
    mode = 0;
  }
  const long long ldd = row_stride_2d(d, "out");
  const int rc = pt_gemm_bf16(a.data_ptr(), b.data_ptr(), d.data_ptr(), (int)M, (int)N, (int)K, lda, ldb, ldd,
                              trans_a ? 1 : 0, trans_b ? 1 : 0, mode, num_sms(), stream());
  TORCH_CHECK(rc == 0, "gemm failed with code ", rc, " (M=", M, " N=", N, " K=", K, " lda=", lda, " ldb=", ldb, " ldd=", ldd,
              " trans_a=", trans_a, " trans_b=", trans_b, " mode=", mode, " a%16=", (uintptr_t)a.data_ptr() % 16,
              " b%16=", (uintptr_t)b.data_ptr() % 16, " d%16=", (uintptr_t)d.data_ptr() % 16, " dev=", (int)a.device().index(), " a_ptr=", (uintptr_t)a.data_ptr(),
              " b_ptr=", (uintptr_t)b.data_ptr(), " a_storage_bytes=", (int64_t)a.storage().nbytes(), ")");
  return d;
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& w, int64_t vocab_start) {
  PT_CHECK_BF16(w);
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && w.is_contiguous());
  c10::cuda::CUDAGuard guard(w.device());
  auto out = torch::empty({ids.numel(), w.size(1)}, w.options());
  PT_CHECK_RC(pt_embedding_fwd((const long long*)ids.data_ptr<int64_t>(), w.data_ptr(), out.data_ptr(), ids.numel(),
                               (int)w.size(1), w.size(0), vocab_start, stream()), "embedding_fwd");
  return out;
}

void embedding_bwd(const Tensor& ids, const Tensor& dy, Tensor& dw, int64_t vocab_start) {
  PT_CHECK_BF16(dy); PT_CHECK_F32(dw);
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && dy.is_contiguous() &&
              dw.is_contiguous() && dy.size(0) == ids.numel() && dy.size(1) == dw.size(1));
  c10::cuda::CUDAGuard guard(dw.device());
  PT_CHECK_RC(pt_embedding_bwd((const long long*)ids.data_ptr<int64_t>(), dy.data_ptr(), dw.data_ptr<float>(),
                               ids.numel(), (int)dw.size(1), dw.size(0), vocab_start, stream()), "embedding_bwd");
}

std::vector<Tensor> ce_stats(const Tensor& logits, const Tensor& targets, int64_t vocab_start) {
  PT_CHECK_BF16(logits);
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() &&
              targets.numel() == logits.size(0));
  const long long ld = row_stride_2d(logits, "logits");
  c10::cuda::CUDAGuard guard(logits.device());
  auto f = logits.options().dtype(at::kFloat);
  auto rowmax = torch::empty({logits.size(0)}, f), sumexp = torch::empty({logits.size(0)}, f),
       tgt = torch::empty({logits.size(0)}, f);
  PT_CHECK_RC(pt_ce_stats(logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(), rowmax.data_ptr<float>(),
                          sumexp.data_ptr<float>(), tgt.data_ptr<float>(), logits.size(0), (int)logits.size(1), ld,
                          vocab_start, stream()), "ce_stats");
  return {rowmax, sumexp, tgt};
}

// logits[T, V] = x w^T together with the cross-entropy row statistics, which the GEMM's epilogue computes tile by tile:
// returns {logits, rowmax, sumexp, target_logit} (the contract of ce_stats), or {} when the fused kernel does not apply.
std::vector<Tensor> gemm_ce_stats(const Tensor& x, const Tensor& w, const Tensor& targets, int64_t vocab_start) {
  PT_CHECK_BF16(x); PT_CHECK_BF16(w);
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == x.size(0));
  const long long lda = row_stride_2d(x, "x"), ldb = row_stride_2d(w, "w");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "gemm_ce_stats: shape mismatch");
  if (!pt_gemm_get_pair() || N % 8 != 0) return {};
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t tiles = (N + 255) / 256;
  auto f = x.options().dtype(at::kFloat);
  auto logits = torch::empty({M, N}, x.options());
  auto part = torch::empty({M, tiles, 2}, f);
  auto tgt = torch::zeros({M}, f);
  const int rc = pt_gemm_bf16_ce(x.data_ptr(), w.data_ptr(), logits.data_ptr(), (int)M, (int)N, (int)K, lda, ldb, N,
                                 (const long long*)targets.data_ptr<int64_t>(), vocab_start, part.data_ptr(),
                                 tgt.data_ptr<float>(), pt_status_word(), stream());
  if (rc == 1 || rc == -5) return {};
  TORCH_CHECK(rc == 0, "gemm_ce_stats failed with code ", rc);
  auto rowmax = torch::empty({M}, f), sumexp = torch::empty({M}, f);
  PT_CHECK_RC(pt_ce_combine(part.data_ptr(), rowmax.data_ptr<float>(), sumexp.data_ptr<float>(), M, (int)tiles, stream()),
              "ce_combine");
  return {logits, rowmax, sumexp, tgt};
}

void ce_grad_(Tensor& logits, const Tensor& targets, const Tensor& lse, double scale, int64_t vocab_start) {
  PT_CHECK_BF16(logits); PT_CHECK_F32(lse);
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() &&
              lse.is_contiguous() && lse.numel() == logits.size(0));
  const long long ld = row_stride_2d(logits, "logits");
  c10::cuda::CUDAGuard guard(logits.device());
  PT_CHECK_RC(pt_ce_grad(logits.data_ptr(), (const long long*)targets.data_ptr<int64_t>(), lse.data_ptr<float>(),
                         logits.size(0), (int)logits.size(1), ld, (float)scale, vocab_start, stream()), "ce_grad");
}

void accumulate_(Tensor& acc, const Tensor& g) {
  PT_CHECK_F32(acc);
  TORCH_CHECK(g.is_cuda() && acc.is_contiguous() && g.is_contiguous() && acc.numel() == g.numel());
  TORCH_CHECK(g.scalar_type() == at::kBFloat16 || g.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(acc.device());
  PT_CHECK_RC(pt_accumulate(acc.data_ptr<float>(), g.data_ptr(), acc.numel(), g.scalar_type() == at::kFloat, stream()),
              "accumulate");
}

Tensor add(const Tensor& a, const Tensor& b) {
  PT_CHECK_BF16(a); PT_CHECK_BF16(b);
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && a.sizes() == b.sizes());
  c10::cuda::CUDAGuard guard(a.device());
  auto out = torch::empty_like(a);
  PT_CHECK_RC(pt_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), stream()), "add");
  return out;
}

void adamw_multi_(std::vector<Tensor> params, std::vector<Tensor> grads, std::vector<Tensor> ms, std::vector<Tensor> vs,
                  std::vector<c10::optional<Tensor>> masters, int64_t step, double lr, double beta1, double beta2,
                  double eps, double wd) {
  const size_t n = params.size();
  TORCH_CHECK(grads.size() == n && ms.size() == n && vs.size() == n && masters.size() == n);
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(params[0].device());
  // group by parameter dtype (bf16 / fp32); everything else must be fp32 and contiguous
  for (int pass = 0; pass < 2; ++pass) {
    const auto want = pass == 0 ? at::kBFloat16 : at::kFloat;
    std::vector<void*> p; std::vector<const float*> g; std::vector<float*> m, v, mw; std::vector<long long> numel;
    for (size_t i = 0; i < n; ++i) {
      if (params[i].scalar_type() != want) continue;
      TORCH_CHECK(params[i].is_cuda() && params[i].is_contiguous() && grads[i].is_contiguous() &&
                  ms[i].is_contiguous() && vs[i].is_contiguous(), "adamw: tensors must be contiguous CUDA tensors");
      PT_CHECK_F32(grads[i]); PT_CHECK_F32(ms[i]); PT_CHECK_F32(vs[i]);
      TORCH_CHECK(grads[i].numel() == params[i].numel() && ms[i].numel() == params[i].numel() &&
                  vs[i].numel() == params[i].numel());
      p.push_back(params[i].data_ptr()); g.push_back(grads[i].data_ptr<float>());
      m.push_back(ms[i].data_ptr<float>()); v.push_back(vs[i].data_ptr<float>());
      if (masters[i].has_value()) { PT_CHECK_F32(*masters[i]); mw.push_back(masters[i]->data_ptr<float>()); }
      else mw.push_back(nullptr);
      numel.push_back(params[i].numel());
    }
    if (p.empty()) continue;
    PT_CHECK_RC(pt_adamw_multi(p.data(), g.data(), m.data(), v.data(), mw.data(), numel.data(), (int)p.size(),
                               pass == 0 ? 1 : 0, (int)step, (float)lr, (float)beta1, (float)beta2, (float)eps,
                               (float)wd, stream()), "adamw_multi");
  }
  for (size_t i = 0; i < n; ++i)
    TORCH_CHECK(params[i].scalar_type() == at::kBFloat16 || params[i].scalar_type() == at::kFloat,
                "adamw: parameters must be bf16 or fp32");
}

void merge_attention_(Tensor& out, Tensor& lse, const Tensor& bo, const Tensor& bl) {
  PT_CHECK_F32(out); PT_CHECK_F32(lse); PT_CHECK_BF16(bo); PT_CHECK_F32(bl);
  TORCH_CHECK(out.dim() == 4 && out.is_contiguous() && bo.is_contiguous() && bo.sizes() == out.sizes() &&
              lse.is_contiguous() && bl.is_contiguous() && lse.sizes() == bl.sizes());
  c10::cuda::CUDAGuard guard(out.device());
  PT_CHECK_RC(pt_merge_attention(out.data_ptr<float>(), lse.data_ptr<float>(), bo.data_ptr(), bl.data_ptr<float>(),
                                 (int)out.size(0), (int)out.size(1), (int)out.size(2), (int)out.size(3), stream()),
              "merge_attention");
}

// q [B,Sq,hq,d], k/v [B,Sk,hkv,d]: last two dims contiguous, token stride arbitrary (slices of packed qkv).
inline long long token_stride(const Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() == 4 && t.stride(3) == 1 && t.stride(2) == t.size(3), name, ": head/feature dims must be packed");
  TORCH_CHECK(t.size(0) == 1 || t.stride(0) == t.stride(1) * t.size(1), name, ": batch and sequence must be collapsible");
  return t.stride(1);
}

std::vector<Tensor> attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, bool causal, double scale) {
  PT_CHECK_BF16(q); PT_CHECK_BF16(k); PT_CHECK_BF16(v);
  const int B = (int)q.size(0), Sq = (int)q.size(1), hq = (int)q.size(2), d = (int)q.size(3);
  const int Sk = (int)k.size(1), hkv = (int)k.size(2);
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && v.size(1) == Sk && v.size(2) == hkv && k.size(3) == d &&
              v.size(3) == d && hq % hkv == 0);
  c10::cuda::CUDAGuard guard(q.device());
  auto o = torch::empty({B, Sq, hq, d}, q.options());
  auto lse = torch::empty({B, hq, Sq}, q.options().dtype(at::kFloat));
  PT_CHECK_RC(pt_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), B, Sq, Sk,
                               hq, hkv, d, token_stride(q, "q"), token_stride(k, "k"), token_stride(v, "v"),
                               causal ? 1 : 0, (float)scale, stream()), "attention_fwd");
  return {o, lse};
}

// With `rope_cos` / `rope_sin` (fp32 [S, d/2]) the inverse rotation of RoPE is applied to dq and dk before they are written
// (query / key i at position i % S), i.e. the gradients are those of the un-rotated q and k.
std::vector<Tensor> attention_bwd(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                  const Tensor& lse, bool causal, double scale, const c10::optional<Tensor>& delta,
                                  const c10::optional<std::vector<Tensor>>& outs, const c10::optional<Tensor>& rope_cos,
                                  const c10::optional<Tensor>& rope_sin) {
  PT_CHECK_BF16(dout); PT_CHECK_BF16(q); PT_CHECK_BF16(k); PT_CHECK_BF16(v); PT_CHECK_BF16(o); PT_CHECK_F32(lse);
  const int B = (int)q.size(0), Sq = (int)q.size(1), hq = (int)q.size(2), d = (int)q.size(3);
  const int Sk = (int)k.size(1), hkv = (int)k.size(2);
  TORCH_CHECK(dout.is_contiguous() && o.is_contiguous() && lse.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  Tensor dq, dk, dv;
  if (outs.has_value()) {
    TORCH_CHECK(outs->size() == 3);
    dq = (*outs)[0]; dk = (*outs)[1]; dv = (*outs)[2];
    PT_CHECK_BF16(dq); PT_CHECK_BF16(dk); PT_CHECK_BF16(dv);
  } else {
    dq = torch::empty({B, Sq, hq, d}, q.options());
    dk = torch::empty({B, Sk, hkv, d}, q.options());
    dv = torch::empty({B, Sk, hkv, d}, q.options());
  }
  auto f = q.options().dtype(at::kFloat);
  Tensor delta_ws = torch::empty({B, hq, Sq}, f);
  Tensor dq_ws = torch::zeros({B, Sq, hq, d}, f);
  if (delta.has_value()) { PT_CHECK_F32(*delta); TORCH_CHECK(delta->is_contiguous() && delta->numel() == delta_ws.numel()); }
  const float* cosp = nullptr;
  const float* sinp = nullptr;
  int rope_seq = 0;
  if (rope_cos.has_value()) {
    TORCH_CHECK(rope_sin.has_value(), "attention_bwd: rope_cos without rope_sin");
    PT_CHECK_F32(*rope_cos); PT_CHECK_F32(*rope_sin);
    TORCH_CHECK(rope_cos->is_contiguous() && rope_sin->is_contiguous() && rope_cos->dim() == 2 && rope_cos->size(1) == d / 2 &&
                rope_sin->sizes() == rope_cos->sizes() && rope_cos->size(0) >= Sq && rope_cos->size(0) >= Sk,
                "attention_bwd: rope tables must be fp32 [S, d/2] with S >= the sequence lengths");
    cosp = rope_cos->data_ptr<float>();
    sinp = rope_sin->data_ptr<float>();
    TORCH_CHECK(Sq == Sk, "attention_bwd: rope fusion needs self-attention (Sq == Sk)");
    rope_seq = Sq;                       // row b*Sq + i of the flattened tokens is at position i
  }
  PT_CHECK_RC(pt_attention_bwd_rope(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                    lse.data_ptr<float>(), delta.has_value() ? delta->data_ptr<float>() : nullptr,
                                    delta_ws.data_ptr<float>(), dq_ws.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(),
                                    dv.data_ptr(), B, Sq, Sk, hq, hkv, d, token_stride(q, "q"), token_stride(k, "k"),
                                    token_stride(v, "v"), token_stride(dq, "dq"), token_stride(dk, "dk"),
                                    token_stride(dv, "dv"), causal ? 1 : 0, (float)scale, cosp, sinp, rope_seq, stream()),
              "attention_bwd");
  return {dq, dk, dv};
}

void allreduce_symm(std::vector<int64_t> buf_ptrs, std::vector<int64_t> flag_ptrs, int64_t mc_ptr, int64_t offset_elems,
                    int64_t n, bool is_bf16, double scale, int64_t rank, int64_t world, int64_t num_blocks,
                    int64_t staging_off_bytes) {
  TORCH_CHECK((int64_t)buf_ptrs.size() == world && (int64_t)flag_ptrs.size() == world && world <= 8);
  void* b[8]; void* f[8];
  for (int i = 0; i < world; ++i) { b[i] = reinterpret_cast<void*>(buf_ptrs[i]); f[i] = reinterpret_cast<void*>(flag_ptrs[i]); }
  PT_CHECK_RC(pt_allreduce_symm(b, f, reinterpret_cast<void*>(mc_ptr), offset_elems, n, is_bf16 ? 1 : 0, (float)scale,
                                (int)rank, (int)world, (int)num_blocks, staging_off_bytes, stream()), "allreduce_symm");
}

// Attention of local queries over K/V segments given by raw (possibly peer-mapped) pointers: segment i is a
// [B, Sk, hkv, d] bf16 tensor with token stride kv_row at k_ptrs[i] / v_ptrs[i]; causal masks inside the last segment.
std::vector<Tensor> attention_fwd_segs(const Tensor& q, std::vector<int64_t> k_ptrs, std::vector<int64_t> v_ptrs, int64_t Sk,
                                       int64_t hkv, int64_t kv_row, bool causal, double scale) {
  PT_CHECK_BF16(q);
  const int B = (int)q.size(0), Sq = (int)q.size(1), hq = (int)q.size(2), d = (int)q.size(3);
  const int n = (int)k_ptrs.size();
  TORCH_CHECK(n >= 1 && n <= 8 && (int)v_ptrs.size() == n);
  c10::cuda::CUDAGuard guard(q.device());
  const void* kp[8]; const void* vp[8];
  for (int i = 0; i < n; ++i) { kp[i] = reinterpret_cast<const void*>(k_ptrs[i]); vp[i] = reinterpret_cast<const void*>(v_ptrs[i]); }
  auto o = torch::empty({B, Sq, hq, d}, q.options());
  auto lse = torch::empty({B, hq, Sq}, q.options().dtype(at::kFloat));
  PT_CHECK_RC(pt_attention_fwd_segs(q.data_ptr(), kp, vp, n, o.data_ptr(), lse.data_ptr<float>(), B, Sq, (int)Sk, hq, (int)hkv,
                                    d, token_stride(q, "q"), kv_row, kv_row, causal ? 1 : 0, (float)scale, stream()),
              "attention_fwd_segs");
  return {o, lse};
}

// Backward of attention_fwd_segs. Returns dq (bf16, contiguous). The fp32 dk/dv partials of segment i are written to
// partial_ptr + i*seg_stride (dk) and + i*seg_stride + B*Sk*hkv*d (dv), token stride hkv*d.
Tensor attention_bwd_segs(const Tensor& dout, const Tensor& q, std::vector<int64_t> k_ptrs, std::vector<int64_t> v_ptrs,
                          int64_t Sk, int64_t hkv, int64_t kv_row, const Tensor& o, const Tensor& lse,
                          const c10::optional<Tensor>& delta, int64_t partial_ptr, int64_t seg_stride, bool causal,
                          double scale) {
  PT_CHECK_BF16(dout); PT_CHECK_BF16(q); PT_CHECK_BF16(o); PT_CHECK_F32(lse);
  if (delta.has_value()) { PT_CHECK_F32(*delta); }
  const int B = (int)q.size(0), Sq = (int)q.size(1), hq = (int)q.size(2), d = (int)q.size(3);
  const int n = (int)k_ptrs.size();
  TORCH_CHECK(n >= 1 && n <= 8 && (int)v_ptrs.size() == n && dout.is_contiguous() && o.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  const void* kp[8]; const void* vp[8];
  for (int i = 0; i < n; ++i) { kp[i] = reinterpret_cast<const void*>(k_ptrs[i]); vp[i] = reinterpret_cast<const void*>(v_ptrs[i]); }
  auto dq = torch::empty({B, Sq, hq, d}, q.options());
  auto dq_ws = torch::zeros({B, Sq, hq, d}, q.options().dtype(at::kFloat));
  auto delta_ws = torch::empty({B, hq, Sq}, q.options().dtype(at::kFloat));
  float* part = reinterpret_cast<float*>(partial_ptr);
  const long long per = (long long)B * Sk * hkv * d;
  PT_CHECK_RC(pt_attention_bwd_segs(dout.data_ptr(), q.data_ptr(), kp, vp, n, o.data_ptr(), lse.data_ptr<float>(),
                                    delta.has_value() ? delta->data_ptr<float>() : nullptr, delta_ws.data_ptr<float>(),
                                    dq_ws.data_ptr<float>(), dq.data_ptr(), part, part + per,
                                    1, seg_stride, B, Sq, (int)Sk, hq, (int)hkv, d, token_stride(q, "q"), kv_row, kv_row,
                                    (long long)hq * d, (long long)hkv * d, (long long)hkv * d, causal ? 1 : 0, (float)scale,
                                    stream()), "attention_bwd_segs");
  return dq;
}

// out (2-D bf16 inside the symmetric data region, element offset d_offset) = sum over ranks of op(a) op(b)
void gemm_allreduce(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b, Tensor& out, std::vector<int64_t> buf_ptrs,
                    std::vector<int64_t> flag_ptrs, int64_t mc_ptr, int64_t d_offset, int64_t rank, int64_t world,
                    int64_t clusters_cap) {
  PT_CHECK_BF16(a); PT_CHECK_BF16(b); PT_CHECK_BF16(out);
  const long long lda = row_stride_2d(a, "a"), ldb = row_stride_2d(b, "b"), ldd = row_stride_2d(out, "out");
  const int64_t M = trans_a ? a.size(1) : a.size(0), K = trans_a ? a.size(0) : a.size(1);
  const int64_t N = trans_b ? b.size(1) : b.size(0), Kb = trans_b ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb && out.size(0) == M && out.size(1) == N, "gemm_allreduce: shape mismatch");
  TORCH_CHECK((int64_t)buf_ptrs.size() == world && (int64_t)flag_ptrs.size() == world && world <= 8);
  c10::cuda::CUDAGuard guard(a.device());
  void* bp[8]; void* fp[8];
  for (int i = 0; i < world; ++i) { bp[i] = reinterpret_cast<void*>(buf_ptrs[i]); fp[i] = reinterpret_cast<void*>(flag_ptrs[i]); }
  const int rc = pt_gemm_allreduce_bf16(a.data_ptr(), b.data_ptr(), bp, fp, reinterpret_cast<void*>(mc_ptr), d_offset, (int)M, (int)N, (int)K, lda, ldb, ldd,
                                        trans_a ? 1 : 0, trans_b ? 1 : 0, (int)rank, (int)world,
                                        (int)clusters_cap, stream());
  TORCH_CHECK(rc == 0, "gemm_allreduce failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
}

// number of CTA pairs of the fused GEMM+all-reduce kernel that fit on the current device
int64_t gemm_allreduce_max_clusters() {
  static const uint16_t dummy[64] = {0};
  void* none[1] = {nullptr};
  const int rc = pt_gemm_allreduce_bf16(dummy, dummy, none, none, nullptr, 0, 256, 256, 64, 64, 64, 256, 0, 0, 0, 1, 0, stream());
  return rc;
}

void symm_barrier(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t world) {
  TORCH_CHECK((int64_t)flag_ptrs.size() == world && world <= 8);
  void* f[8];
  for (int i = 0; i < world; ++i) f[i] = reinterpret_cast<void*>(flag_ptrs[i]);
  PT_CHECK_RC(pt_symm_barrier(f, (int)rank, (int)world, stream()), "symm_barrier");
}

void reduce_dkv_symm(std::vector<int64_t> buf_ptrs, int64_t offset_elems, int64_t me, int64_t world, Tensor& dk, Tensor& dv) {
  PT_CHECK_BF16(dk); PT_CHECK_BF16(dv);
  TORCH_CHECK((int64_t)buf_ptrs.size() == world && world <= 8 && dk.dim() == 4 && dk.sizes() == dv.sizes());
  c10::cuda::CUDAGuard guard(dk.device());
  void* b[8];
  for (int i = 0; i < world; ++i) b[i] = reinterpret_cast<void*>(buf_ptrs[i]);
  const long long tokens = dk.size(0) * dk.size(1);
  const int width = (int)(dk.size(2) * dk.size(3));
  PT_CHECK_RC(pt_reduce_dkv_symm(b, offset_elems, (int)me, (int)world, tokens, width, dk.data_ptr(), dv.data_ptr(),
                                 token_stride(dk, "dk"), token_stride(dv, "dv"), stream()), "reduce_dkv_symm");
}

// out[T, H] (bf16): row ids[t] of a vocabulary-parallel embedding whose shards ([rows_per_rank, H] each) are at shard_ptrs
Tensor embedding_gather_peers(const Tensor& ids, std::vector<int64_t> shard_ptrs, int64_t rows_per_rank, int64_t H, const Tensor& like) {
  PT_CHECK_BF16(like);
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && shard_ptrs.size() >= 1 && shard_ptrs.size() <= 8);
  c10::cuda::CUDAGuard guard(like.device());
  void* b[8];
  for (size_t i = 0; i < shard_ptrs.size(); ++i) b[i] = reinterpret_cast<void*>(shard_ptrs[i]);
  auto out = torch::empty({ids.numel(), H}, like.options());
  PT_CHECK_RC(pt_embedding_gather_peers((const long long*)ids.data_ptr<int64_t>(), b, (int)shard_ptrs.size(), rows_per_rank,
                                        ids.numel(), (int)H, out.data_ptr(), stream()), "embedding_gather_peers");
  return out;
}

// {lse, target_logit} of n rows from the per-shard statistics every rank of the group left at `offset_bytes` of its buffer
std::vector<Tensor> ce_stats_combine_peers(std::vector<int64_t> buf_ptrs, int64_t offset_bytes, int64_t n, const Tensor& like) {
  TORCH_CHECK(buf_ptrs.size() >= 1 && buf_ptrs.size() <= 8 && like.is_cuda());
  c10::cuda::CUDAGuard guard(like.device());
  void* b[8];
  for (size_t i = 0; i < buf_ptrs.size(); ++i) b[i] = reinterpret_cast<void*>(buf_ptrs[i]);
  auto f = like.options().dtype(at::kFloat);
  auto lse = torch::empty({n}, f), tgt = torch::empty({n}, f);
  PT_CHECK_RC(pt_ce_stats_combine_peers(b, offset_bytes, (int)buf_ptrs.size(), n, lse.data_ptr<float>(), tgt.data_ptr<float>(),
                                        stream()), "ce_stats_combine_peers");
  return {lse, tgt};
}

// dst (contiguous, n blocks of bytes_each) <- the blocks at src_ptrs (raw, possibly peer-mapped device pointers)
void gather_peer(Tensor& dst, std::vector<int64_t> src_ptrs, int64_t bytes_each) {
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && src_ptrs.size() <= 8);
  TORCH_CHECK((int64_t)(dst.numel() * dst.element_size()) >= bytes_each * (int64_t)src_ptrs.size(), "gather_peer: dst too small");
  c10::cuda::CUDAGuard guard(dst.device());
  const void* p[8];
  for (size_t i = 0; i < src_ptrs.size(); ++i) p[i] = reinterpret_cast<const void*>(src_ptrs[i]);
  PT_CHECK_RC(pt_gather_peer(dst.data_ptr(), p, (int)src_ptrs.size(), bytes_each, stream()), "gather_peer");
}

int64_t kernel_status() { return (int64_t)pt_kernel_status_fetch_and_clear(); }
int64_t launch_count() { return (int64_t)pt_launch_count(); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"), py::arg("dres") = py::none(),
        py::arg("dw_acc") = py::none());
  m.def("rope_", &rope_);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("trans_a"), py::arg("trans_b"), py::arg("out") = py::none(),
        py::arg("accumulate") = false);
  m.def("gemm_swiglu", &gemm_swiglu, "x w_gu^T with the SwiGLU activation fused into the GEMM epilogue: returns [gu, h] or [].");
  m.def("gemm_rope", &gemm_rope, "x w_qkv^T with RoPE of the first n_rot heads fused into the GEMM epilogue (None if not covered).");
  m.def("gemm_add", &gemm_add, "x w^T + res with the residual add fused into the GEMM epilogue (None if not covered).");
  m.def("gemm_dgrad_swiglu_bwd", &gemm_dgrad_swiglu_bwd,
        "SwiGLU backward fused into the epilogue of the down-projection dgrad GEMM: returns the packed [T, 2I] gradient (None if not covered).");
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("ce_stats", &ce_stats);
  m.def("gemm_ce_stats", &gemm_ce_stats,
        "LM-head GEMM whose epilogue also produces the cross-entropy row statistics: [logits, rowmax, sumexp, target_logit] or [].");
  m.def("ce_grad_", &ce_grad_);
  m.def("accumulate_", &accumulate_);
  m.def("add", &add);
  m.def("adamw_multi_", &adamw_multi_);
  m.def("merge_attention_", &merge_attention_);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd, py::arg("dout"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"),
        py::arg("lse"), py::arg("causal"), py::arg("scale"), py::arg("delta") = py::none(), py::arg("outs") = py::none(),
        py::arg("rope_cos") = py::none(), py::arg("rope_sin") = py::none());
  m.def("set_gemm_pair", [](bool on) { pt_gemm_set_pair(on ? 1 : 0); },
        "Use 256x256 tiles on CTA pairs (tcgen05 cta_group::2) for GEMMs (default) or 128x256 single-CTA tiles.");
  m.def("get_gemm_pair", []() { return pt_gemm_get_pair() != 0; });
  m.def("set_gemm_tma_epilogue", [](bool on) { pt_gemm_set_tma_epilogue(on ? 1 : 0); },
        "CTA-pair GEMM epilogue through shared memory and TMA store / reduce-add (default) or per-thread 16-byte stores.");
  m.def("get_gemm_tma_epilogue", []() { return pt_gemm_get_tma_epilogue() != 0; });
  m.def("set_gemm_group_m", [](int64_t g) { pt_gemm_set_group_m((int)g); },
        "CTA-pair GEMM tile numbering: rows of 256-row tiles per group (L2 locality of concurrently running tiles; default 8).");
  m.def("get_gemm_group_m", []() { return (int64_t)pt_gemm_get_group_m(); });
  m.def("attention_set_profile", [](const c10::optional<Tensor>& counters) {
          if (!counters.has_value()) { pt_attention_set_profile(nullptr); return; }
          TORCH_CHECK(counters->is_cuda() && counters->scalar_type() == at::kLong && counters->is_contiguous() &&
                      counters->numel() >= 16, "attention_set_profile: need a contiguous CUDA int64 tensor of >= 16 elements");
          pt_attention_set_profile(reinterpret_cast<unsigned long long*>(counters->data_ptr<int64_t>()));
        }, py::arg("counters") = py::none(),
        "Phase profiling of the attention kernels: later forward/backward launches add their per-phase SM-cycle counts to "
        "`counters` (layout in csrc/attention_tcgen05.cu); None switches it off. The caller keeps the tensor alive.");
  m.def("attention_fwd_segs", &attention_fwd_segs);
  m.def("attention_bwd_segs", &attention_bwd_segs);
  m.def("gemm_allreduce", &gemm_allreduce,
        "GEMM whose output tiles are all-reduced over peer memory inside the same kernel (csrc/gemm_allreduce_tcgen05.cu).");
  m.def("gemm_allreduce_max_clusters", &gemm_allreduce_max_clusters);
  m.def("symm_barrier", &symm_barrier);
  m.def("reduce_dkv_symm", &reduce_dkv_symm);
  m.def("embedding_gather_peers", &embedding_gather_peers,
        "Vocabulary-parallel embedding lookup that reads every row from its owner's shard in symmetric memory (no reduction).");
  m.def("ce_stats_combine_peers", &ce_stats_combine_peers,
        "Vocabulary-parallel cross entropy: combine the per-shard (max, sum-exp, target logit) triples of all ranks (csrc/comm.cu).");
  m.def("gather_peer", &gather_peer, "Copy equally sized blocks out of peers' memory into one local buffer (csrc/comm.cu).");
  m.def("allreduce_symm", &allreduce_symm,
        "In-place all-reduce of a region of a symmetric buffer over peer memory (see csrc/comm.cu).");
  m.def("set_pdl", [](bool on) { pt_set_pdl(on ? 1 : 0); },
        "Programmatic dependent launch of the step's kernels (prologues overlap the previous kernel's tail); default on, "
        "PICOTRON_PDL=0 switches it off.");
  m.def("get_pdl", []() { return pt_pdl_enabled() != 0; });
  m.def("set_wait_limit_ns", [](int64_t ns) { pt_set_wait_limit_ns((unsigned long long)(ns > 0 ? ns : 0)); },
        "Limit (ns of the GPU global timer) of every cross-rank wait inside the peer-memory kernels; 0 restores the default (4 s). "
        "A wait that runs out makes the kernel return early and leaves a code in the status word (kernel_status).");
  m.def("get_wait_limit_ns", []() { return (int64_t)pt_get_wait_limit_ns(); });
  m.def("count_launches", [](int64_t n) { pt_count_launches((int)n); },
        "Add n to the launch counter (kernels replayed from a CUDA graph are launched without passing through this library).");
  m.def("launch_count", &launch_count, "Number of kernels this library has launched in this process.");
  m.def("kernel_status", &kernel_status,
        "Fetch-and-clear the device status word: 0 if no kernel gave up a bounded wait, else an encoded site.");
}
