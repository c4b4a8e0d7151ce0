// Memory-bound kernels of the model: RMSNorm (+residual) fwd/bwd, RoPE, SwiGLU, embedding, cross-entropy
// statistics/gradient, fp32 gradient accumulation, multi-tensor AdamW, attention-partial merge, add.
//
// They replace, for sm_100a, the Triton/ATen kernels the reference reaches (picotron/model.py:54-65 RMSNorm,
// :136-137 RoPE, :186 SiLU*mul, :251 embedding; train.py:46-49 cross entropy; data_parallel.py:131 grad
// accumulation; train.py:209,235 AdamW; context_parallel.py:157-187 LSE merge).
// All of them are bandwidth-bound: 16-byte vector accesses, fp32 math, one pass over HBM per tensor.
#include "common.cuh"
#include "noalloc.h"

namespace pt {

typedef __nv_bfloat16 bf16;

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm: block size and column chunks per thread of the partial-sum backward below (H % 8 == 0, H <= 8 * THREADS * MAXC)
// ---------------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXC = 4;

// ---------------------------------------------------------------------------------------------
// RMSNorm backward. dx = rstd * (w*dy - xhat * mean(xhat * w*dy)) (+ dres);  dw = sum_rows dy * xhat.
// A persistent grid walks the rows; every CTA keeps its dw partial in registers and writes it to
// `partial[grid, H]` (scratch), a second kernel sums the partials.
// ---------------------------------------------------------------------------------------------
template <int MAXC>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                   const float* __restrict__ rstd_in, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                   float* __restrict__ partial, int T, int H) {
  __shared__ float red[32];
  const int nchunk = H / 8;
  float wv[MAXC][8];
  float dwacc[MAXC][8];
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (c < nchunk) unpack8(*reinterpret_cast<const bf16x8*>(w + c * 8), wv[i]);
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float xh[MAXC][8], wdy[MAXC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) {
        float xv[8], dv[8];
        unpack8(*reinterpret_cast<const bf16x8*>(x + row * H + c * 8), xv);
        unpack8(*reinterpret_cast<const bf16x8*>(dy + row * H + c * 8), dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xv[j] * rstd;
          wdy[i][j] = dv[j] * wv[i][j];
          dot += xh[i][j] * wdy[i][j];
          dwacc[i][j] += dv[j] * xh[i][j];
        }
      }
    }
    dot = block_sum<NORM_THREADS>(dot, red);
    const float cmean = dot / (float)H;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (wdy[i][j] - xh[i][j] * cmean) * rstd;
        if (dres != nullptr) {
          float r[8];
          unpack8(*reinterpret_cast<const bf16x8*>(dres + row * H + c * 8), r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        *reinterpret_cast<bf16x8*>(dx + row * H + c * 8) = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nchunk) {
      float4* dst = reinterpret_cast<float4*>(partial + (long long)blockIdx.x * H + c * 8);
      dst[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      dst[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// out[col] = sum_p partial[p, col]. Block = 32 columns x 8 row-slices; grid = ceil(H / 32).
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int nparts, int H) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (col < H)
    for (int p = ry; p < nparts; p += 8) s += partial[(long long)p * H + col];
  red[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && col < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i][cx];
    out[col] = t;
  }
}

// ---------------------------------------------------------------------------------------------
// RoPE, NeoX (half-split) layout, in place on the first n_rot heads of every row of a packed
// [T, row_stride] activation. cos/sin: fp32 [S, d/2]. Row t is at position t % S.
// One thread handles 8 consecutive elements of the first half and their partners in the second half.
// ---------------------------------------------------------------------------------------------
__global__ void rope_kernel(bf16* __restrict__ qkv, const float* __restrict__ cosT, const float* __restrict__ sinT,
                            long long total, int n_rot, int d, int S, long long row_stride, float sign) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int half = d / 2;
  const int cpp = half / 8;  // chunks per head
  const int c = (int)(idx % cpp);
  const long long hr = idx / cpp;
  const int head = (int)(hr % n_rot);
  const long long row = hr / n_rot;
  const int pos = (int)(row % S);
  bf16* p1 = qkv + row * row_stride + (long long)head * d + c * 8;
  bf16* p2 = p1 + half;
  float a[8], b[8], cs[8], sn[8];
  unpack8(*reinterpret_cast<const bf16x8*>(p1), a);
  unpack8(*reinterpret_cast<const bf16x8*>(p2), b);
  const float4* c4 = reinterpret_cast<const float4*>(cosT + (long long)pos * half + c * 8);
  const float4* s4 = reinterpret_cast<const float4*>(sinT + (long long)pos * half + c * 8);
  float4 t;
  t = c4[0]; cs[0] = t.x; cs[1] = t.y; cs[2] = t.z; cs[3] = t.w;
  t = c4[1]; cs[4] = t.x; cs[5] = t.y; cs[6] = t.z; cs[7] = t.w;
  t = s4[0]; sn[0] = t.x; sn[1] = t.y; sn[2] = t.z; sn[3] = t.w;
  t = s4[1]; sn[4] = t.x; sn[5] = t.y; sn[6] = t.z; sn[7] = t.w;
  float o1[8], o2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float s = sn[j] * sign;
    o1[j] = a[j] * cs[j] - b[j] * s;
    o2[j] = b[j] * cs[j] + a[j] * s;
  }
  *reinterpret_cast<bf16x8*>(p1) = pack8(o1);
  *reinterpret_cast<bf16x8*>(p2) = pack8(o2);
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on packed [T, 2I] pre-activations (gate | up)
// ---------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long long total8, int I8) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const long long row = idx / I8;
  const int c = (int)(idx % I8);
  const bf16* g = gu + row * (long long)(I8 * 16) + c * 8;
  float gv[8], uv[8], o[8];
  unpack8(*reinterpret_cast<const bf16x8*>(g), gv);
  unpack8(*reinterpret_cast<const bf16x8*>(g + I8 * 8), uv);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sig = 1.f / (1.f + __expf(-gv[j]));
    o[j] = gv[j] * sig * uv[j];
  }
  *reinterpret_cast<bf16x8*>(out + row * (long long)(I8 * 8) + c * 8) = pack8(o);
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ da, bf16* __restrict__ dgu,
                                  long long total8, int I8) {
  pdl_enter();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const long long row = idx / I8;
  const int c = (int)(idx % I8);
  const long long off = row * (long long)(I8 * 16) + c * 8;
  float gv[8], uv[8], dv[8], dg[8], du[8];
  unpack8(*reinterpret_cast<const bf16x8*>(gu + off), gv);
  unpack8(*reinterpret_cast<const bf16x8*>(gu + off + I8 * 8), uv);
  unpack8(*reinterpret_cast<const bf16x8*>(da + row * (long long)(I8 * 8) + c * 8), dv);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sig = 1.f / (1.f + __expf(-gv[j]));
    const float silu = gv[j] * sig;
    dg[j] = dv[j] * uv[j] * (sig * (1.f + gv[j] * (1.f - sig)));
    du[j] = dv[j] * silu;
  }
  *reinterpret_cast<bf16x8*>(dgu + off) = pack8(dg);
  *reinterpret_cast<bf16x8*>(dgu + off + I8 * 8) = pack8(du);
}

// ---------------------------------------------------------------------------------------------
// (vocab-parallel) embedding: rows for ids in [vocab_start, vocab_start + rows), zeros otherwise
// ---------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ w,
                                     bf16* __restrict__ out, int H8, long long rows, long long vocab_start) {
  pdl_enter();
  const long long tok = blockIdx.x;
  const long long id = ids[tok] - vocab_start;
  const bool ok = id >= 0 && id < rows;
  const uint4* src = reinterpret_cast<const uint4*>(w + (ok ? id : 0) * (long long)(H8 * 8));
  uint4* dst = reinterpret_cast<uint4*>(out + tok * (long long)(H8 * 8));
  for (int c = threadIdx.x; c < H8; c += blockDim.x) dst[c] = ok ? src[c] : make_uint4(0, 0, 0, 0);
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ dy,
                                     float* __restrict__ dw, int H8, long long rows, long long vocab_start) {
  pdl_enter();
  const long long tok = blockIdx.x;
  const long long id = ids[tok] - vocab_start;
  if (id < 0 || id >= rows) return;
  float* dst = dw + id * (long long)(H8 * 8);
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    float v[8];
    unpack8(*reinterpret_cast<const bf16x8*>(dy + tok * (long long)(H8 * 8) + c * 8), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + c * 8 + j, v[j]);
  }
}

// ---------------------------------------------------------------------------------------------
// cross entropy over a (shard of the) vocabulary: row statistics, then the in-place gradient
// ---------------------------------------------------------------------------------------------
constexpr int CE_THREADS = 512;

__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const bf16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ rowmax,
                float* __restrict__ sumexp, float* __restrict__ tgt, int V, long long ld, long long vocab_start) {
  __shared__ float red_m[32], red_s[32];
  pdl_enter();
  const long long row = blockIdx.x;
  const bf16* l = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  const int nchunk = (ld % 8 == 0) ? V / 8 : 0;  // rows are 16-byte aligned only when ld is a multiple of 8
  for (int c = threadIdx.x; c < nchunk; c += CE_THREADS) {
    float v[8];
    unpack8(*reinterpret_cast<const bf16x8*>(l + c * 8), v);
    float cm = v[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, v[j]);
    const float nm = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(v[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nchunk * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    const float v = __bfloat162float(l[i]);
    const float nm = fmaxf(m, v);
    s = s * __expf(m - nm) + __expf(v - nm);
    m = nm;
  }
  // merge (m, s) pairs: warp, then block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red_m[warp] = m;
    red_s[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < CE_THREADS / 32 ? red_m[lane] : -INFINITY;
    s = lane < CE_THREADS / 32 ? red_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    if (lane == 0) {
      rowmax[row] = m;
      sumexp[row] = s;
      const long long t = targets[row] - vocab_start;
      tgt[row] = (t >= 0 && t < V) ? __bfloat162float(l[t]) : 0.f;
    }
  }
}

__global__ void __launch_bounds__(CE_THREADS)
ce_grad_kernel(bf16* __restrict__ logits, const long long* __restrict__ targets, const float* __restrict__ lse,
               int V, long long ld, float scale, long long vocab_start) {
  pdl_enter();
  const long long row = blockIdx.x;
  bf16* l = logits + row * ld;
  const float z = lse[row];
  const long long t = targets[row] - vocab_start;
  const int nchunk = (ld % 8 == 0) ? V / 8 : 0;
  for (int c = threadIdx.x; c < nchunk; c += CE_THREADS) {
    float v[8];
    unpack8(*reinterpret_cast<const bf16x8*>(l + c * 8), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(v[j] - z);
      if ((long long)(c * 8 + j) == t) p -= 1.f;
      v[j] = p * scale;
    }
    *reinterpret_cast<bf16x8*>(l + c * 8) = pack8(v);
  }
  for (int i = nchunk * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    float p = __expf(__bfloat162float(l[i]) - z);
    if ((long long)i == t) p -= 1.f;
    l[i] = __float2bfloat16(p * scale);
  }
}

// ---------------------------------------------------------------------------------------------
// fp32 += bf16 ; bf16 add
// ---------------------------------------------------------------------------------------------
__global__ void accumulate_kernel(float* __restrict__ acc, const bf16* __restrict__ g, long long n) {
  const long long i8 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 + 8 <= n) {
    float v[8];
    unpack8(*reinterpret_cast<const bf16x8*>(g + i8), v);
    float4* a = reinterpret_cast<float4*>(acc + i8);
    float4 a0 = a[0], a1 = a[1];
    a0.x += v[0]; a0.y += v[1]; a0.z += v[2]; a0.w += v[3];
    a1.x += v[4]; a1.y += v[5]; a1.z += v[6]; a1.w += v[7];
    a[0] = a0;
    a[1] = a1;
  } else {
    for (long long i = i8; i < n; ++i) acc[i] += __bfloat162float(g[i]);
  }
}

__global__ void accumulate_f32_kernel(float* __restrict__ acc, const float* __restrict__ g, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) acc[i] += g[i];
}

__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ out, long long n) {
  pdl_enter();
  const long long i8 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 + 8 <= n) {
    float x[8], y[8];
    unpack8(*reinterpret_cast<const bf16x8*>(a + i8), x);
    unpack8(*reinterpret_cast<const bf16x8*>(b + i8), y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    *reinterpret_cast<bf16x8*>(out + i8) = pack8(x);
  } else {
    for (long long i = i8; i < n; ++i) out[i] = __float2bfloat16(__bfloat162float(a[i]) + __bfloat162float(b[i]));
  }
}

// ---------------------------------------------------------------------------------------------
// multi-tensor AdamW (decoupled weight decay), fp32 gradients, fp32 or bf16 moments, optional fp32 master
// ---------------------------------------------------------------------------------------------
constexpr int ADAM_MAX_TENSORS = 24;
constexpr int ADAM_MAX_BLOCKS = 320;
constexpr int ADAM_CHUNK = 65536;

struct AdamArgs {
  void* param[ADAM_MAX_TENSORS];
  const float* grad[ADAM_MAX_TENSORS];
  float* m[ADAM_MAX_TENSORS];
  float* v[ADAM_MAX_TENSORS];
  float* master[ADAM_MAX_TENSORS];
  long long numel[ADAM_MAX_TENSORS];
  unsigned char block_tensor[ADAM_MAX_BLOCKS];
  int block_chunk[ADAM_MAX_BLOCKS];
};

template <bool PARAM_BF16>
__global__ void __launch_bounds__(512)
adamw_kernel(const __grid_constant__ AdamArgs args, float lr, float beta1, float beta2, float eps, float wd,
             float bc1, float bc2_sqrt) {
  const int ti = args.block_tensor[blockIdx.x];
  const long long base = (long long)args.block_chunk[blockIdx.x] * ADAM_CHUNK;
  const long long n = args.numel[ti];
  const float* g = args.grad[ti];
  float* m = args.m[ti];
  float* v = args.v[ti];
  float* mw = args.master[ti];
  for (long long i = base + threadIdx.x; i < base + ADAM_CHUNK && i < n; i += blockDim.x) {
    float w;
    if (mw != nullptr) w = mw[i];
    else if (PARAM_BF16) w = __bfloat162float(reinterpret_cast<bf16*>(args.param[ti])[i]);
    else w = reinterpret_cast<float*>(args.param[ti])[i];
    const float gi = g[i];
    const float mi = m[i] * beta1 + gi * (1.f - beta1);
    const float vi = v[i] * beta2 + gi * gi * (1.f - beta2);
    w = w * (1.f - lr * wd);
    w -= (lr / bc1) * (mi / (sqrtf(vi) / bc2_sqrt + eps));
    m[i] = mi;
    v[i] = vi;
    if (mw != nullptr) mw[i] = w;
    if (PARAM_BF16) reinterpret_cast<bf16*>(args.param[ti])[i] = __float2bfloat16(w);
    else reinterpret_cast<float*>(args.param[ti])[i] = w;
  }
}

// ---------------------------------------------------------------------------------------------
// merge of two attention partials (ring attention): out fp32 [B,S,h,d], lse fp32 [B,h,S]
//   out -= sigmoid(bl - l) * (out - block_out);   l -= logsigmoid(l - bl)
// ---------------------------------------------------------------------------------------------
__global__ void merge_attention_kernel(float* __restrict__ out, float* __restrict__ lse, const bf16* __restrict__ bo,
                                       const float* __restrict__ bl, int B, int S, int h, int d) {
  // one warp per (b, s, head)
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * h;
  if (wid >= total) return;
  const int head = (int)(wid % h);
  const long long bs = wid / h;
  const int s = (int)(bs % S);
  const int b = (int)(bs / S);
  const long long li = ((long long)b * h + head) * S + s;
  const float l = lse[li], nb = bl[li];
  const float sig = 1.f / (1.f + __expf(l - nb));          // sigmoid(nb - l)
  float* o = out + wid * d;
  const bf16* n = bo + wid * d;
  for (int j = lane; j < d; j += 32) o[j] -= sig * (o[j] - __bfloat162float(n[j]));
  __syncwarp();
  if (lane == 0) {
    // l - logsigmoid(l - nb) = l + log(1 + exp(nb - l)) computed stably
    const float mx = fmaxf(l, nb);
    lse[li] = mx + __logf(__expf(l - mx) + __expf(nb - mx));
  }
}

}  // namespace pt

// ===============================================================================================
// C launch API (raw pointers; the Python bindings validate shapes and dtypes)
// ===============================================================================================
using namespace pt;

extern "C" void pt_count_launches(int n);
static inline int check_launch(int n = 1) {
  pt_count_launches(n);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------------------------
// Row-block RMSNorm kernels (the ones the training step runs). A CTA of 256 threads owns fixed columns -- thread t
// holds the 16-byte chunks t, t + 256, ... of a row -- and walks the rows R at a time: all loads of the R rows are
// issued before the first reduction, the R row sums are reduced together (one CTA barrier per R rows, double-buffered
// scratch), and because the columns of a thread never change, the weight and the weight-gradient accumulators live
// in registers for the whole kernel. (One CTA per row forward and one warp per row backward, which these replace, reached
// 0.3-0.4 of the copy bandwidth: every row was a load -> reduce -> store chain with nothing else in flight in that warp.)
//   forward :  x_new = x (+ delta); rstd = rsqrt(mean(x_new^2) + eps); y = x_new * rstd * w
//   backward:  dx = rstd * (w*dy - xhat * mean(xhat*w*dy)) (+ dres);  dw_acc += sum_rows dy * xhat   (fp32 reductions)
// H % 8 == 0, H <= 8 * 256 * NC.
// ---------------------------------------------------------------------------------------------
constexpr int ROWS_THREADS = 256;

// sums[r] over the CTA for r < R; `red` is [2][R][8] floats, `it` alternates the half that is written
template <int R>
__device__ __forceinline__ void block_sum_rows(float (&v)[R], float* red, int it) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = red + (it & 1) * R * 8;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    v[r] = warp_sum(v[r]);
    if (lane == 0) buf[r * 8 + warp] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float4 a = *reinterpret_cast<const float4*>(buf + r * 8), b = *reinterpret_cast<const float4*>(buf + r * 8 + 4);
    v[r] = (a.x + a.y) + (a.z + a.w) + (b.x + b.y) + (b.z + b.w);
  }
}

template <bool ADD, int NC, int R>
__global__ void __launch_bounds__(ROWS_THREADS)
rmsnorm_fwd_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ delta, const bf16* __restrict__ w,
                        bf16* __restrict__ x_new, bf16* __restrict__ y, float* __restrict__ rstd_out, int T, int H, float eps) {
  __shared__ __align__(16) float red[2 * R * 8];
  pdl_enter();
  const int nchunk = H / 8;
  bf16x8 wv[NC];
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    const int c = threadIdx.x + i * ROWS_THREADS;
    if (c < nchunk) wv[i] = *reinterpret_cast<const bf16x8*>(w + c * 8);
  }
  int it = 0;
  for (long long row0 = (long long)blockIdx.x * R; row0 < T; row0 += (long long)gridDim.x * R, ++it) {
    bf16x8 px[R][NC], pd[R][NC];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = threadIdx.x + i * ROWS_THREADS;
        if (row0 + r < T && c < nchunk) {
          px[r][i] = *reinterpret_cast<const bf16x8*>(x + (row0 + r) * H + c * 8);
          if (ADD) pd[r][i] = *reinterpret_cast<const bf16x8*>(delta + (row0 + r) * H + c * 8);
        }
      }
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      ss[r] = 0.f;
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = threadIdx.x + i * ROWS_THREADS;
        if (row0 + r < T && c < nchunk) {
          float v[8];
          unpack8(px[r][i], v);
          if (ADD) {
            float d[8];
            unpack8(pd[r][i], d);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += d[j];
            px[r][i] = pack8(v);                       // the rounded residual stream is what the backward sees
            *reinterpret_cast<bf16x8*>(x_new + (row0 + r) * H + c * 8) = px[r][i];
            unpack8(px[r][i], v);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) ss[r] += v[j] * v[j];
        }
      }
    }
    block_sum_rows<R>(ss, red, it);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= T) continue;
      const float rstd = rsqrtf(ss[r] / (float)H + eps);
      if (threadIdx.x == 0) rstd_out[row0 + r] = rstd;
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = threadIdx.x + i * ROWS_THREADS;
        if (c < nchunk) {
          float v[8], ww[8], o[8];
          unpack8(px[r][i], v);
          unpack8(wv[i], ww);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[j] * rstd * ww[j];
          *reinterpret_cast<bf16x8*>(y + (row0 + r) * H + c * 8) = pack8(o);
        }
      }
    }
  }
}

template <int NC, int R>
__global__ void __launch_bounds__(ROWS_THREADS)
rmsnorm_bwd_rows_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                        const float* __restrict__ rstd_in, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                        float* __restrict__ dw_acc, int T, int H) {
  __shared__ __align__(16) float red[2 * R * 8];
  pdl_enter();
  const int nchunk = H / 8;
  bf16x8 wv[NC];
  float dwacc[NC][8];
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    const int c = threadIdx.x + i * ROWS_THREADS;
    if (c < nchunk) wv[i] = *reinterpret_cast<const bf16x8*>(w + c * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  }
  int it = 0;
  for (long long row0 = (long long)blockIdx.x * R; row0 < T; row0 += (long long)gridDim.x * R, ++it) {
    bf16x8 px[R][NC], pdy[R][NC], pr[R][NC];
    float rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      rstd[r] = row0 + r < T ? rstd_in[row0 + r] : 0.f;
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = threadIdx.x + i * ROWS_THREADS;
        if (row0 + r < T && c < nchunk) {
          px[r][i] = *reinterpret_cast<const bf16x8*>(x + (row0 + r) * H + c * 8);
          pdy[r][i] = *reinterpret_cast<const bf16x8*>(dy + (row0 + r) * H + c * 8);
          if (dres != nullptr) pr[r][i] = *reinterpret_cast<const bf16x8*>(dres + (row0 + r) * H + c * 8);
        }
      }
    }
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      dot[r] = 0.f;
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = threadIdx.x + i * ROWS_THREADS;
        if (row0 + r < T && c < nchunk) {
          float xv[8], dv[8], ww[8];
          unpack8(px[r][i], xv);
          unpack8(pdy[r][i], dv);
          unpack8(wv[i], ww);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = xv[j] * rstd[r];
            dot[r] += xh * dv[j] * ww[j];
            dwacc[i][j] += dv[j] * xh;
          }
        }
      }
    }
    block_sum_rows<R>(dot, red, it);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= T) continue;
      const float cmean = dot[r] / (float)H;
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = threadIdx.x + i * ROWS_THREADS;
        if (c < nchunk) {
          float xv[8], dv[8], ww[8], o[8];
          unpack8(px[r][i], xv);
          unpack8(pdy[r][i], dv);
          unpack8(wv[i], ww);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (dv[j] * ww[j] - xv[j] * rstd[r] * cmean) * rstd[r];
          if (dres != nullptr) {
            float rr[8];
            unpack8(pr[r][i], rr);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += rr[j];
          }
          *reinterpret_cast<bf16x8*>(dx + (row0 + r) * H + c * 8) = pack8(o);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    const int c = threadIdx.x + i * ROWS_THREADS;
    if (c < nchunk) {
      float* dst = dw_acc + c * 8;
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(dwacc[i][0]), "f"(dwacc[i][1]),
                   "f"(dwacc[i][2]), "f"(dwacc[i][3]) : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(dwacc[i][4]), "f"(dwacc[i][5]),
                   "f"(dwacc[i][6]), "f"(dwacc[i][7]) : "memory");
    }
  }
}

// grid of a row-block kernel: every CTA gets work, at most `per_sm` CTAs per SM
static inline int rows_grid(int T, int R, int num_sms, int per_sm) {
  const int want = (T + R - 1) / R, cap = num_sms * per_sm;
  return want < cap ? want : cap;
}

extern "C" int pt_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* x_new, void* y, float* rstd,
                              int T, int H, float eps, cudaStream_t st) {
  if (H % 8 || H > 8 * ROWS_THREADS * 4) return -10;
  if (T == 0) return 0;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int nc = (H / 8 + ROWS_THREADS - 1) / ROWS_THREADS;
#define PT_NORM_FWD(ADD, NC, R)                                                                                      \
  launch_pdl(rmsnorm_fwd_rows_kernel<ADD, NC, R>, dim3(rows_grid(T, R, num_sms, 4)), dim3(ROWS_THREADS), 0, st,      \
             (const bf16*)x, (const bf16*)delta, (const bf16*)w, (bf16*)x_new, (bf16*)y, rstd, T, H, eps)
  if (delta != nullptr) {
    if (nc <= 1) PT_NORM_FWD(true, 1, 4); else if (nc <= 2) PT_NORM_FWD(true, 2, 2); else PT_NORM_FWD(true, 4, 1);
  } else {
    if (nc <= 1) PT_NORM_FWD(false, 1, 4); else if (nc <= 2) PT_NORM_FWD(false, 2, 2); else PT_NORM_FWD(false, 4, 1);
  }
#undef PT_NORM_FWD
  return check_launch();
}

// number of dw partial rows the backward needs in `partial` ([rows, H] fp32 scratch)
extern "C" int pt_rmsnorm_bwd_partial_rows(int T, int num_sms) {
  int g = 4 * num_sms;
  return T < g ? T : g;
}

static void launch_rmsnorm_bwd(int grid, const void* dy, const void* x, const void* w, const float* rstd,
                               const void* dres, void* dx, float* partial, int T, int H, cudaStream_t st) {
  const int mc = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define PT_NORM_BWD(MC)                                                                                      \
  rmsnorm_bwd_kernel<MC><<<grid, NORM_THREADS, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, \
                                                        (const bf16*)dres, (bf16*)dx, partial, T, H)
  if (mc <= 1) PT_NORM_BWD(1); else if (mc <= 2) PT_NORM_BWD(2); else PT_NORM_BWD(4);
#undef PT_NORM_BWD
}

extern "C" int pt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                              void* dx, float* dw, float* partial, int T, int H, int num_sms, cudaStream_t st) {
  if (H % 8 || H > 8 * NORM_THREADS * NORM_MAXC) return -10;
  if (T == 0) return 0;
  const int grid = pt_rmsnorm_bwd_partial_rows(T, num_sms);
  launch_rmsnorm_bwd(grid, dy, x, w, rstd, dres, dx, partial, T, H, st);
  reduce_partials_kernel<<<(H + 31) / 32, 256, 0, st>>>(partial, dw, grid, H);
  return check_launch(2);
}

// RMSNorm backward that ADDS dw into `dw_acc` (fp32 [H], e.g. the weight's gradient-bucket slice) with vector
// reductions instead of writing per-CTA partials and summing them in a second kernel. Summation order of dw is
// not fixed from run to run. Returns 1 (nothing launched) when the shape is not covered: H % 8 != 0, H > 8192 or a
// dw_acc that is not 16-byte aligned.
extern "C" int pt_rmsnorm_bwd_acc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                  void* dx, float* dw_acc, int T, int H, int num_sms, cudaStream_t st) {
  if (H % 8 || H > 8 * ROWS_THREADS * 4 || (reinterpret_cast<uintptr_t>(dw_acc) & 15)) return 1;
  if (T == 0) return 0;
  const int nc = (H / 8 + ROWS_THREADS - 1) / ROWS_THREADS;
#define PT_NORM_BWD_ROWS(NC, R)                                                                                      \
  launch_pdl(rmsnorm_bwd_rows_kernel<NC, R>, dim3(rows_grid(T, R, num_sms, 2)), dim3(ROWS_THREADS), 0, st,           \
             (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)dres, (bf16*)dx, dw_acc, T, H)
  if (nc <= 1) PT_NORM_BWD_ROWS(1, 4); else if (nc <= 2) PT_NORM_BWD_ROWS(2, 2); else PT_NORM_BWD_ROWS(4, 1);
#undef PT_NORM_BWD_ROWS
  return check_launch();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of pt_rmsnorm_bwd (contract in noalloc.h): the dw partials live in a file-scope
// device array instead of a caller-provided scratch buffer. In host code `g_noalloc_partial` is only a
// stand-in for the symbol; its device address is resolved once per device with cudaGetSymbolAddress.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_noalloc_partial[PT_NOALLOC_MAX_ROWS * PT_NOALLOC_MAX_H];
static float* g_noalloc_partial_addr[64] = {nullptr};

extern "C" int pt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                      const void* dres, void* dx, float* dw, int T, int H, cudaStream_t st) {
  if (T <= 0 || H <= 0 || H % 8) return PT_NOALLOC_ERR_BAD_SHAPE;
  if (H > PT_NOALLOC_MAX_H) return PT_NOALLOC_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PT_NOALLOC_ERR_SYMBOL;
  if (g_noalloc_partial_addr[dev] == nullptr) {
    // first call on this device: look the array up while this device is current
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_noalloc_partial) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return PT_NOALLOC_ERR_SYMBOL;
    }
    g_noalloc_partial_addr[dev] = p;
  }
  float* partial = g_noalloc_partial_addr[dev];
  const int grid = T < PT_NOALLOC_MAX_ROWS ? T : PT_NOALLOC_MAX_ROWS;   // one partial row per CTA
  launch_rmsnorm_bwd(grid, dy, x, w, rstd, dres, dx, partial, T, H, st);
  reduce_partials_kernel<<<(H + 31) / 32, 256, 0, st>>>(partial, dw, grid, H);
  return check_launch(2) == 0 ? PT_NOALLOC_OK : PT_NOALLOC_ERR_LAUNCH;
}

extern "C" const char* pt_noalloc_strerror(int code) {
  switch (code) {
    case PT_NOALLOC_OK: return "ok";
    case PT_NOALLOC_ERR_BAD_SHAPE: return "bad shape: T must be positive and H a positive multiple of 8";
    case PT_NOALLOC_ERR_TOO_LARGE: return "problem too large for the built-in scratch array: H exceeds PT_NOALLOC_MAX_H (4096)";
    case PT_NOALLOC_ERR_SYMBOL: return "could not resolve the device address of the built-in scratch array";
    case PT_NOALLOC_ERR_LAUNCH: return "kernel launch failed";
    default: return "unknown code";
  }
}

extern "C" int pt_rope(void* qkv, const float* cosT, const float* sinT, long long T, int n_rot, int d, int S,
                       long long row_stride, int inverse, cudaStream_t st) {
  if (d % 16 || row_stride % 8) return -10;
  const long long total = T * n_rot * (d / 16);
  if (total == 0) return 0;
  rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((bf16*)qkv, cosT, sinT, total, n_rot, d, S, row_stride,
                                                              inverse ? -1.f : 1.f);
  return check_launch();
}

extern "C" int pt_swiglu_fwd(const void* gu, void* out, long long T, int I, cudaStream_t st) {
  if (I % 8) return -10;
  const long long total = T * (I / 8);
  if (total == 0) return 0;
  swiglu_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const bf16*)gu, (bf16*)out, total, I / 8);
  return check_launch();
}

extern "C" int pt_swiglu_bwd(const void* gu, const void* da, void* dgu, long long T, int I, cudaStream_t st) {
  if (I % 8) return -10;
  const long long total = T * (I / 8);
  if (total == 0) return 0;
  launch_pdl(swiglu_bwd_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, (const bf16*)gu, (const bf16*)da,
             (bf16*)dgu, total, I / 8);
  return check_launch();
}

extern "C" int pt_embedding_fwd(const long long* ids, const void* w, void* out, long long T, int H, long long rows,
                                long long vocab_start, cudaStream_t st) {
  if (H % 8) return -10;
  if (T == 0) return 0;
  launch_pdl(embedding_fwd_kernel, dim3((unsigned)T), dim3(256), 0, st, ids, (const bf16*)w, (bf16*)out, H / 8, rows, vocab_start);
  return check_launch();
}

extern "C" int pt_embedding_bwd(const long long* ids, const void* dy, float* dw, long long T, int H, long long rows,
                                long long vocab_start, cudaStream_t st) {
  if (H % 8) return -10;
  if (T == 0) return 0;
  launch_pdl(embedding_bwd_kernel, dim3((unsigned)T), dim3(256), 0, st, ids, (const bf16*)dy, dw, H / 8, rows, vocab_start);
  return check_launch();
}

extern "C" int pt_ce_stats(const void* logits, const long long* targets, float* rowmax, float* sumexp, float* tgt,
                           long long T, int V, long long ld, long long vocab_start, cudaStream_t st) {
  if (T == 0) return 0;
  launch_pdl(ce_stats_kernel, dim3((unsigned)T), dim3(CE_THREADS), 0, st, (const bf16*)logits, targets, rowmax, sumexp, tgt, V, ld,
             vocab_start);
  return check_launch();
}

// Merge the per-tile (max, sum-exp) pairs the LM-head GEMM's epilogue left in part[T, tiles]: one warp per row.
__global__ void __launch_bounds__(256)
ce_combine_kernel(const float2* __restrict__ part, float* __restrict__ rowmax, float* __restrict__ sumexp, long long T, int tiles) {
  pdl_enter();
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  float m = -INFINITY, s = 0.f;
  for (int t = lane; t < tiles; t += 32) {
    const float2 p = part[row * tiles + t];
    const float nm = fmaxf(m, p.x);
    s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + p.y * __expf(p.x - nm);
    m = nm;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  if (lane == 0) {
    rowmax[row] = m;
    sumexp[row] = s;
  }
}

extern "C" int pt_ce_combine(const void* part, float* rowmax, float* sumexp, long long T, int tiles, cudaStream_t st) {
  if (T == 0) return 0;
  launch_pdl(ce_combine_kernel, dim3((unsigned)((T + 7) / 8)), dim3(256), 0, st, (const float2*)part, rowmax, sumexp, T, tiles);
  return check_launch();
}

extern "C" int pt_ce_grad(void* logits, const long long* targets, const float* lse, long long T, int V, long long ld,
                          float scale, long long vocab_start, cudaStream_t st) {
  if (T == 0) return 0;
  launch_pdl(ce_grad_kernel, dim3((unsigned)T), dim3(CE_THREADS), 0, st, (bf16*)logits, targets, lse, V, ld, scale, vocab_start);
  return check_launch();
}

extern "C" int pt_accumulate(float* acc, const void* g, long long n, int g_is_f32, cudaStream_t st) {
  if (n == 0) return 0;
  if (g_is_f32)
    accumulate_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(acc, (const float*)g, n);
  else
    accumulate_kernel<<<(unsigned)((n / 8 + 1 + 255) / 256), 256, 0, st>>>(acc, (const bf16*)g, n);
  return check_launch();
}

extern "C" int pt_add(const void* a, const void* b, void* out, long long n, cudaStream_t st) {
  if (n == 0) return 0;
  launch_pdl(add_kernel, dim3((unsigned)((n / 8 + 1 + 255) / 256)), dim3(256), 0, st, (const bf16*)a, (const bf16*)b, (bf16*)out, n);
  return check_launch();
}

// AdamW over `count` tensors. params: bf16 (param_is_bf16) or fp32. grads/m/v fp32. masters[i] may be null.
extern "C" int pt_adamw_multi(void** params, const float** grads, float** ms, float** vs, float** masters,
                              const long long* numels, int count, int param_is_bf16, int step, float lr, float beta1,
                              float beta2, float eps, float wd, cudaStream_t st) {
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  AdamArgs args;
  int nt = 0, nb = 0;
  auto flush = [&]() -> int {
    if (nb == 0) return 0;
    if (param_is_bf16)
      adamw_kernel<true><<<nb, 512, 0, st>>>(args, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt);
    else
      adamw_kernel<false><<<nb, 512, 0, st>>>(args, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt);
    nt = nb = 0;
    return check_launch();
  };
  for (int i = 0; i < count; ++i) {
    const long long n = numels[i];
    if (n == 0) continue;
    long long chunks = (n + ADAM_CHUNK - 1) / ADAM_CHUNK;
    long long c0 = 0;
    while (c0 < chunks) {
      if (nt == ADAM_MAX_TENSORS || nb == ADAM_MAX_BLOCKS) {
        if (int rc = flush()) return rc;
      }
      args.param[nt] = params[i];
      args.grad[nt] = grads[i];
      args.m[nt] = ms[i];
      args.v[nt] = vs[i];
      args.master[nt] = masters[i];
      args.numel[nt] = n;
      while (c0 < chunks && nb < ADAM_MAX_BLOCKS) {
        args.block_tensor[nb] = (unsigned char)nt;
        args.block_chunk[nb] = (int)c0;
        ++nb;
        ++c0;
      }
      ++nt;
    }
  }
  return flush();
}

extern "C" int pt_merge_attention(float* out, float* lse, const void* bo, const float* bl, int B, int S, int h, int d,
                                  cudaStream_t st) {
  const long long warps = (long long)B * S * h;
  if (warps == 0) return 0;
  merge_attention_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(out, lse, (const bf16*)bo, bl, B, S, h, d);
  return check_launch();
}
