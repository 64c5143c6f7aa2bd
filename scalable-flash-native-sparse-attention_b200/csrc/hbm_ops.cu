// Memory-bound pieces of the NSA path: window pooling, window gather (im2col), gate activations, the gated
// combine and the context-parallel chunk reorder.  All of them move 16 bytes per thread per access and do
// their arithmetic in fp32.
#include <algorithm>
#include "nsa_common.cuh"

namespace nsa {

struct F8 {
  float v[8];
};
__device__ __forceinline__ F8 unpack8(uint4 u) {
  F8 r;
  r.v[0] = bf16_lo(u.x); r.v[1] = bf16_hi(u.x);
  r.v[2] = bf16_lo(u.y); r.v[3] = bf16_hi(u.y);
  r.v[4] = bf16_lo(u.z); r.v[5] = bf16_hi(u.z);
  r.v[6] = bf16_lo(u.w); r.v[7] = bf16_hi(u.w);
  return r;
}
__device__ __forceinline__ uint4 pack8(const F8& f) {
  uint4 u;
  u.x = pack_bf16(f.v[0], f.v[1]);
  u.y = pack_bf16(f.v[2], f.v[3]);
  u.z = pack_bf16(f.v[4], f.v[5]);
  u.w = pack_bf16(f.v[6], f.v[7]);
  return u;
}
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// ------------------------------------------------------------------------------------------------ pooling
// y[j,h,:] = (sum_{i<ks} x[st*j+i,h,:]) / ks          grid: (cdiv(y_maxlen*CH,256), n_seq, H)
__global__ void mean_pool_fwd_kernel(NsaPoolParams p) {
  const int CH = p.D / 8;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  int j = idx / CH, c = idx % CH;
  int b = blockIdx.y, h = blockIdx.z;
  int x_bos = p.meta.x_cu[b];
  int y_bos = p.meta.y_cu[b], y_len = p.meta.y_cu[b + 1] - y_bos;
  if (j >= y_len) return;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x) +
                           (int64_t)(x_bos + (int64_t)j * p.hp.stride) * p.x_stride_t + h * p.D + c * 8;
  F8 acc;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc.v[e] = 0.f;
  for (int i = 0; i < p.hp.kernel_size; ++i) {
    F8 f = unpack8(ldg16(x + (int64_t)i * p.x_stride_t));
#pragma unroll
    for (int e = 0; e < 8; ++e) acc.v[e] += f.v[e];
  }
  float inv = 1.f / (float)p.hp.kernel_size;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc.v[e] *= inv;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.y) + (int64_t)(y_bos + j) * p.y_stride_t + h * p.D + c * 8;
  *reinterpret_cast<uint4*>(y) = pack8(acc);
}

// dx[t,h,:] (+)= sum over rows j whose window holds t of dy[j,h,:] / ks      grid: (cdiv(x_maxlen*CH,256), n_seq, H)
__global__ void mean_pool_bwd_kernel(NsaPoolParams p) {
  const int CH = p.D / 8;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  int t = idx / CH, c = idx % CH;
  int b = blockIdx.y, h = blockIdx.z;
  int x_bos = p.meta.x_cu[b], x_len = p.meta.x_cu[b + 1] - x_bos;
  int y_bos = p.meta.y_cu[b], y_len = p.meta.y_cu[b + 1] - y_bos;
  if (t >= x_len) return;
  const int ks = p.hp.kernel_size, st = p.hp.stride;
  int j_hi = min(t / st, y_len - 1);
  int j_lo = max((t - ks + st) / st, 0);  // ceil((t-ks+1)/st) for t-ks+1 > 0
  if (t - ks + 1 <= 0) j_lo = 0;
  F8 acc;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc.v[e] = 0.f;
  const __nv_bfloat16* dy = reinterpret_cast<const __nv_bfloat16*>(p.y) + h * p.D + c * 8;
  for (int j = j_lo; j <= j_hi; ++j) {
    F8 f = unpack8(ldg16(dy + (int64_t)(y_bos + j) * p.y_stride_t));
#pragma unroll
    for (int e = 0; e < 8; ++e) acc.v[e] += f.v[e];
  }
  float inv = 1.f / (float)ks;
  float* dx = p.dx + (int64_t)(x_bos + t) * p.dx_stride_t + h * p.D + c * 8;
  float4 o0, o1;
  if (p.accumulate) {
    o0 = *reinterpret_cast<float4*>(dx);
    o1 = *reinterpret_cast<float4*>(dx + 4);
  } else {
    o0 = make_float4(0.f, 0.f, 0.f, 0.f);
    o1 = o0;
  }
  o0.x += acc.v[0] * inv; o0.y += acc.v[1] * inv; o0.z += acc.v[2] * inv; o0.w += acc.v[3] * inv;
  o1.x += acc.v[4] * inv; o1.y += acc.v[5] * inv; o1.z += acc.v[6] * inv; o1.w += acc.v[7] * inv;
  *reinterpret_cast<float4*>(dx) = o0;
  *reinterpret_cast<float4*>(dx + 4) = o1;
}

// ------------------------------------------------------------------------------------------------ im2col
// y[j,h,i,:] = x[st*j+i,h,:]                      grid: (cdiv(y_maxlen*ks*CH,256), n_seq, H)
__global__ void construct_block_fwd_kernel(NsaBlockParams p) {
  const int CH = p.D / 8;
  const int ks = p.hp.kernel_size;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int c = idx % CH;
  int i = (idx / CH) % ks;
  int j = idx / ((int64_t)CH * ks);
  int b = blockIdx.y, h = blockIdx.z;
  int x_bos = p.meta.x_cu[b];
  int y_bos = p.meta.y_cu[b], y_len = p.meta.y_cu[b + 1] - y_bos;
  if (j >= y_len) return;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x) +
                           (int64_t)(x_bos + (int64_t)j * p.hp.stride + i) * p.x_stride_t + h * p.D + c * 8;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.y) +
                     (((int64_t)(y_bos + j) * p.H + h) * ks + i) * p.D + c * 8;
  *reinterpret_cast<uint4*>(y) = ldg16(x);
}

// dx[t,h,:] (+)= sum_j dy[j,h,t-st*j,:]           grid: (cdiv(x_maxlen*CH,256), n_seq, H)
__global__ void construct_block_bwd_kernel(NsaBlockParams p) {
  const int CH = p.D / 8;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  int t = idx / CH, c = idx % CH;
  int b = blockIdx.y, h = blockIdx.z;
  int x_bos = p.meta.x_cu[b], x_len = p.meta.x_cu[b + 1] - x_bos;
  int y_bos = p.meta.y_cu[b], y_len = p.meta.y_cu[b + 1] - y_bos;
  if (t >= x_len) return;
  const int ks = p.hp.kernel_size, st = p.hp.stride;
  int j_hi = min(t / st, y_len - 1);
  int j_lo = (t - ks + 1 <= 0) ? 0 : (t - ks + st) / st;
  F8 acc;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc.v[e] = 0.f;
  const __nv_bfloat16* dy = reinterpret_cast<const __nv_bfloat16*>(p.y);
  for (int j = j_lo; j <= j_hi; ++j) {
    int i = t - st * j;
    F8 f = unpack8(ldg16(dy + (((int64_t)(y_bos + j) * p.H + h) * ks + i) * p.D + c * 8));
#pragma unroll
    for (int e = 0; e < 8; ++e) acc.v[e] += f.v[e];
  }
  float* dx = p.dx + (int64_t)(x_bos + t) * p.dx_stride_t + h * p.D + c * 8;
#pragma unroll
  for (int e = 0; e < 8; ++e) dx[e] = (p.accumulate ? dx[e] : 0.f) + acc.v[e];
}

// ------------------------------------------------------------------------------------------------ gate activations
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void act_fwd_kernel(NsaActParams p) {
  const int CH = p.K / 8;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.M * CH) return;
  int64_t m = idx / CH;
  int c = idx % CH;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x) + m * 2 * p.K + c * 8;
  F8 g = unpack8(ldg16(x)), u = unpack8(ldg16(x + p.K)), y;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float s = sigmoidf_(g.v[e]);
    y.v[e] = (p.kind == 0 ? g.v[e] * s : s) * u.v[e];
  }
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y) + m * p.K + c * 8) = pack8(y);
}

__global__ void act_bwd_kernel(NsaActParams p) {
  const int CH = p.K / 8;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.M * CH) return;
  int64_t m = idx / CH;
  int c = idx % CH;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(p.x) + m * 2 * p.K + c * 8;
  F8 g = unpack8(*reinterpret_cast<const uint4*>(x)), u = unpack8(*reinterpret_cast<const uint4*>(x + p.K));
  F8 dy = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.dy) + m * p.K + c * 8));
  F8 dg, du;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float s = sigmoidf_(g.v[e]);
    if (p.kind == 0) {
      du.v[e] = dy.v[e] * g.v[e] * s;
      dg.v[e] = dy.v[e] * u.v[e] * s * (1.f + g.v[e] * (1.f - s));
    } else {
      du.v[e] = dy.v[e] * s;
      dg.v[e] = dy.v[e] * u.v[e] * s * (1.f - s);
    }
  }
  __nv_bfloat16* dx = reinterpret_cast<__nv_bfloat16*>(p.dx) + m * 2 * p.K + c * 8;
  *reinterpret_cast<uint4*>(dx) = pack8(dg);
  *reinterpret_cast<uint4*>(dx + p.K) = pack8(du);
}

// ------------------------------------------------------------------------------------------------ gated combine
// one thread per 8 output elements; the D/8 threads of a (t,h) row are adjacent lanes of one warp
__global__ void combine_fwd_kernel(NsaCombineParams p) {
  const int CH = p.D / 8;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t row = idx / CH;
  int c = idx % CH;
  if (row >= p.T * p.H) return;
  int64_t t = row / p.H;
  int h = row % p.H;
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(p.w) + t * p.w_stride_t + h * 3;
  float s0 = sigmoidf_(__bfloat162float(w[0])), s1 = sigmoidf_(__bfloat162float(w[1])),
        s2 = sigmoidf_(__bfloat162float(w[2]));
  int64_t col = (int64_t)h * p.D + c * 8;
  F8 a = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.a) + t * p.a_stride_t + col));
  F8 b = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.b) + t * p.b_stride_t + col));
  F8 cc = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.c) + t * p.c_stride_t + col));
  F8 y;
#pragma unroll
  for (int e = 0; e < 8; ++e) y.v[e] = a.v[e] * s0 + b.v[e] * s1 + cc.v[e] * s2;
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y) + t * p.y_stride_t + col) = pack8(y);
}

__global__ void combine_bwd_kernel(NsaCombineParams p) {
  const int CH = p.D / 8;  // 8 or 16: a row's threads are an aligned lane group
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t row = idx / CH;
  int c = idx % CH;
  bool live = row < p.T * p.H;
  int64_t t = live ? row / p.H : 0;
  int h = live ? row % p.H : 0;
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(p.w) + t * p.w_stride_t + h * 3;
  float s0 = sigmoidf_(__bfloat162float(w[0])), s1 = sigmoidf_(__bfloat162float(w[1])),
        s2 = sigmoidf_(__bfloat162float(w[2]));
  int64_t col = (int64_t)h * p.D + c * 8;
  F8 a = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.a) + t * p.a_stride_t + col));
  F8 b = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.b) + t * p.b_stride_t + col));
  F8 cc = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.c) + t * p.c_stride_t + col));
  F8 dy = unpack8(ldg16(reinterpret_cast<const __nv_bfloat16*>(p.dy) + t * p.dy_stride_t + col));
  F8 da, db, dc;
  float r0 = 0.f, r1 = 0.f, r2 = 0.f;
  float d0 = 0.f, d1 = 0.f, d2 = 0.f;   // delta of each branch, from the bf16-rounded branch gradients that are stored
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    da.v[e] = dy.v[e] * s0;
    db.v[e] = dy.v[e] * s1;
    dc.v[e] = dy.v[e] * s2;
    r0 += dy.v[e] * a.v[e];
    r1 += dy.v[e] * b.v[e];
    r2 += dy.v[e] * cc.v[e];
    d0 += __bfloat162float(__float2bfloat16(da.v[e])) * a.v[e];
    d1 += __bfloat162float(__float2bfloat16(db.v[e])) * b.v[e];
    d2 += __bfloat162float(__float2bfloat16(dc.v[e])) * cc.v[e];
  }
  for (int o = CH / 2; o > 0; o >>= 1) {
    r0 += __shfl_xor_sync(0xffffffffu, r0, o);
    r1 += __shfl_xor_sync(0xffffffffu, r1, o);
    r2 += __shfl_xor_sync(0xffffffffu, r2, o);
    d0 += __shfl_xor_sync(0xffffffffu, d0, o);
    d1 += __shfl_xor_sync(0xffffffffu, d1, o);
    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
  }
  if (!live) return;
  int64_t ocol = (t * p.H + h) * (int64_t)p.D + c * 8;  // da/db/dc are contiguous [T,H,D]
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.da) + ocol) = pack8(da);
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.db) + ocol) = pack8(db);
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.dc) + ocol) = pack8(dc);
  if (c == 0) {
    __nv_bfloat16* dw = reinterpret_cast<__nv_bfloat16*>(p.dw) + t * p.dw_stride_t + h * 3;
    dw[0] = __float2bfloat16(s0 * (1.f - s0) * r0);
    dw[1] = __float2bfloat16(s1 * (1.f - s1) * r1);
    dw[2] = __float2bfloat16(s2 * (1.f - s2) * r2);
    if (p.delta_a) {
      p.delta_a[t * p.delta_a_stride_t + h * p.delta_a_stride_h] = d0;
      p.delta_b[t * p.delta_b_stride_t + h * p.delta_b_stride_h] = d1;
      p.delta_c[t * p.delta_c_stride_t + h * p.delta_c_stride_h] = d2;
    }
  }
}

// ------------------------------------------------------------------------------------------------ cache store
__global__ void store_kvcache_kernel(NsaStoreKvParams p) {
  const int CH = p.row_elems / 8;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t n = idx / CH;
  if (n >= p.N) return;
  const int c = (int)(idx - n * CH);
  const int slot = __ldg(p.slot_mapping + n);
  if (slot < 0) return;
  const __nv_bfloat16* ks = reinterpret_cast<const __nv_bfloat16*>(p.key) + n * p.key_stride + c * 8;
  const __nv_bfloat16* vs = reinterpret_cast<const __nv_bfloat16*>(p.value) + n * p.value_stride + c * 8;
  const int64_t off = (int64_t)slot * p.row_elems + c * 8;
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.k_cache) + off) = ldg16(ks);
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.v_cache) + off) = ldg16(vs);
}

// ------------------------------------------------------------------------------------------------ rotary embedding
// One thread = 8 elements of the first half of a head and the matching 8 of the second half, for q heads then k heads of
// one (batch, position) row; cos / sin are read once per thread (16 B each half).  In place is safe: a thread reads
// both halves before it writes either.
__global__ void rope_kernel(NsaRopeParams p) {
  const int HC = p.D / 16;                       // 16-byte chunks per half head
  const int per_row = (p.QH + p.KH) * HC;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = idx / per_row;
  if (row >= (int64_t)p.B * p.N) return;
  const int r = (int)(idx - row * per_row);
  const int hh = r / HC, c = r - hh * HC;
  const int64_t b = row / p.N, n = row - b * p.N;
  const bool is_k = hh >= p.QH;
  const int h = is_k ? hh - p.QH : hh;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(is_k ? p.k : p.q) +
                           (is_k ? b * p.k_stride_b + n * p.k_stride_n + h * p.k_stride_h : b * p.q_stride_b + n * p.q_stride_n + h * p.q_stride_h);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(is_k ? p.ke : p.qe) +
                     (is_k ? b * p.ke_stride_b + n * p.ke_stride_n + h * p.ke_stride_h : b * p.qe_stride_b + n * p.qe_stride_n + h * p.qe_stride_h);
  const int64_t co = b * p.cos_stride_b + n * p.cos_stride_n;
  const __nv_bfloat16* cs = reinterpret_cast<const __nv_bfloat16*>(p.cos) + co;
  const __nv_bfloat16* sn = reinterpret_cast<const __nv_bfloat16*>(p.sin) + co;
  const int half = p.D / 2, o1 = c * 8, o2 = half + c * 8;
  const F8 x1 = unpack8(ldg16(x + o1)), x2 = unpack8(ldg16(x + o2));
  const F8 c1 = unpack8(ldg16(cs + o1)), c2 = unpack8(ldg16(cs + o2));
  const F8 s1 = unpack8(ldg16(sn + o1)), s2 = unpack8(ldg16(sn + o2));
  F8 e1, e2;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    if (!p.backward) {
      e1.v[e] = x1.v[e] * c1.v[e] - x2.v[e] * s1.v[e];
      e2.v[e] = x2.v[e] * c2.v[e] + x1.v[e] * s2.v[e];
    } else {   // x1, x2 are the gradients of e1, e2
      e1.v[e] = x1.v[e] * c1.v[e] + x2.v[e] * s2.v[e];
      e2.v[e] = x2.v[e] * c2.v[e] - x1.v[e] * s1.v[e];
    }
  }
  *reinterpret_cast<uint4*>(y + o1) = pack8(e1);
  *reinterpret_cast<uint4*>(y + o2) = pack8(e2);
}

// ------------------------------------------------------------------------------------------------ chunk reorder
// "shuffle": sequential chunk m < W goes to slot 2m, chunk m+W goes to slot 2(W-m)-1 ... i.e. slot 2i holds
// chunk i and slot 2i+1 holds chunk 2W-1-i.  "unshuffle" is the inverse.
__global__ void reorder_kernel(NsaReorderParams p) {
  int64_t per = p.chunk_bytes / 16;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= per * 2 * p.world_size) return;
  int slot = idx / per;
  int64_t within = idx % per;
  int chunk = (slot & 1) ? (2 * p.world_size - 1 - slot / 2) : slot / 2;  // slot (rank-major) -> sequential chunk
  int src = p.unshuffle ? slot : chunk;
  int dst = p.unshuffle ? chunk : slot;
  const uint4* x = reinterpret_cast<const uint4*>(p.x);
  uint4* y = reinterpret_cast<uint4*>(p.y);
  y[dst * per + within] = x[src * per + within];
}

// ------------------------------------------------------------------------------------------------ paged pooling
// prefill: grid (cdiv(y_maxlen*CH,256), B, H*ncache); decode: grid (cdiv(CH,32)... one thread per 16 B of the row
__global__ void paged_pool_kernel(NsaPagedPoolParams p) {
  const int CH = p.D / 8;
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  int j = idx / CH, c = idx % CH;
  const int b = blockIdx.y;
  const int h = blockIdx.z % p.H;
  __nv_bfloat16* cache = reinterpret_cast<__nv_bfloat16*>(blockIdx.z / p.H ? p.cache1 : p.cache0);
  int slot;
  if (p.decode) {
    if (j > 0) return;
    slot = p.slot_mapping[b];
    if (slot < 0) return;
    int x_len = p.context_lens[b];
    if (x_len <= p.kernel_size - 1) return;
    j = (x_len - p.kernel_size) / p.stride;
  } else {
    int y_bos = p.y_cu[b], y_len = p.y_cu[b + 1] - y_bos;
    if (j >= y_len) return;
    slot = p.slot_mapping[y_bos + j];
    if (slot < 0) return;
  }
  const int32_t* tab = p.kv_table + (int64_t)b * p.table_stride;
  F8 acc;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc.v[e] = 0.f;
  const int start = j * p.stride;
  // rows are added in order; eight of them are fetched together (page-table entry, then the row: two dependent memory
  // round trips that a one-row-at-a-time loop pays kernel_size times)
  for (int i0 = 0; i0 < p.kernel_size; i0 += 8) {
    uint4 piece[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = start + min(i0 + u, p.kernel_size - 1);
      const int64_t row = (int64_t)tab[r / p.page_size] * p.page_size + r % p.page_size;
      piece[u] = *reinterpret_cast<const uint4*>(cache + row * p.row_stride + h * p.D + c * 8);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (i0 + u < p.kernel_size) {
        const F8 f = unpack8(piece[u]);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc.v[e] += f.v[e];
      }
    }
  }
  float inv = 1.f / (float)p.kernel_size;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc.v[e] *= inv;
  *reinterpret_cast<uint4*>(cache + (int64_t)slot * p.row_stride + h * p.D + c * 8) = pack8(acc);
}

// ------------------------------------------------------------------------------------------------ delta = rowsum(o*do)
// one thread per 8 elements of a (t,h) row; used by every attention backward.
__global__ void delta_kernel(const __nv_bfloat16* o, const __nv_bfloat16* dout, float* delta, int64_t T, int H, int D,
                             int64_t o_stride_t, int64_t do_stride_t, int64_t lse_stride_t, int64_t lse_stride_h) {
  const int CH = D / 8;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t row = idx / CH;
  int c = idx % CH;
  bool live = row < T * H;
  int64_t t = live ? row / H : 0;
  int h = live ? row % H : 0;
  int64_t col = (int64_t)h * D + c * 8;
  F8 a = unpack8(ldg16(o + t * o_stride_t + col));
  F8 b = unpack8(ldg16(dout + t * do_stride_t + col));
  float r = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) r += a.v[e] * b.v[e];
  for (int off = CH / 2; off > 0; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
  if (live && c == 0) delta[t * lse_stride_t + h * lse_stride_h] = r;
}

void launch_delta(const void* o, const void* dout, float* delta, int64_t T, int H, int D, int64_t o_stride_t,
                  int64_t do_stride_t, int64_t lse_stride_t, int64_t lse_stride_h, cudaStream_t st) {
  int64_t n = T * H * (D / 8);
  if (n == 0) return;
  delta_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(o),
                                                            reinterpret_cast<const __nv_bfloat16*>(dout), delta, T, H, D,
                                                            o_stride_t, do_stride_t, lse_stride_t, lse_stride_h);
}

}  // namespace nsa

using namespace nsa;

extern "C" int nsa_mean_pool_fwd(const NsaPoolParams* p, void* stream) {
  NSA_REQUIRE(p && p->x && p->y && p->meta.x_cu && p->meta.y_cu, NSA_ERR_BAD_ARG, "mean_pool_fwd: null pointer");
  NSA_REQUIRE(p->D % 8 == 0 && p->D > 0, NSA_ERR_UNSUPPORTED_SHAPE, "mean_pool_fwd: D=%d must be a multiple of 8", p->D);
  if (p->meta.y_maxlen <= 0 || p->meta.n_seq <= 0) return NSA_OK;
  dim3 grid((unsigned)(((int64_t)p->meta.y_maxlen * (p->D / 8) + 255) / 256), p->meta.n_seq, p->H);
  mean_pool_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("mean_pool_fwd");
}

extern "C" int nsa_mean_pool_bwd(const NsaPoolParams* p, void* stream) {
  NSA_REQUIRE(p && p->y && p->dx && p->meta.x_cu && p->meta.y_cu, NSA_ERR_BAD_ARG, "mean_pool_bwd: null pointer");
  NSA_REQUIRE(p->D % 8 == 0 && p->D > 0, NSA_ERR_UNSUPPORTED_SHAPE, "mean_pool_bwd: D=%d must be a multiple of 8", p->D);
  if (p->meta.x_maxlen <= 0 || p->meta.n_seq <= 0) return NSA_OK;
  dim3 grid((unsigned)(((int64_t)p->meta.x_maxlen * (p->D / 8) + 255) / 256), p->meta.n_seq, p->H);
  mean_pool_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("mean_pool_bwd");
}

extern "C" int nsa_construct_block_fwd(const NsaBlockParams* p, void* stream) {
  NSA_REQUIRE(p && p->x && p->y && p->meta.x_cu && p->meta.y_cu, NSA_ERR_BAD_ARG, "construct_block_fwd: null pointer");
  NSA_REQUIRE(p->D % 8 == 0 && p->D > 0, NSA_ERR_UNSUPPORTED_SHAPE, "construct_block_fwd: D=%d", p->D);
  if (p->meta.y_maxlen <= 0 || p->meta.n_seq <= 0) return NSA_OK;
  int64_t n = (int64_t)p->meta.y_maxlen * p->hp.kernel_size * (p->D / 8);
  dim3 grid((unsigned)((n + 255) / 256), p->meta.n_seq, p->H);
  construct_block_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("construct_block_fwd");
}

extern "C" int nsa_construct_block_bwd(const NsaBlockParams* p, void* stream) {
  NSA_REQUIRE(p && p->y && p->dx && p->meta.x_cu && p->meta.y_cu, NSA_ERR_BAD_ARG, "construct_block_bwd: null pointer");
  NSA_REQUIRE(p->D % 8 == 0 && p->D > 0, NSA_ERR_UNSUPPORTED_SHAPE, "construct_block_bwd: D=%d", p->D);
  if (p->meta.x_maxlen <= 0 || p->meta.n_seq <= 0) return NSA_OK;
  dim3 grid((unsigned)(((int64_t)p->meta.x_maxlen * (p->D / 8) + 255) / 256), p->meta.n_seq, p->H);
  construct_block_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("construct_block_bwd");
}

extern "C" int nsa_act_fwd(const NsaActParams* p, void* stream) {
  NSA_REQUIRE(p && p->x && p->y, NSA_ERR_BAD_ARG, "act_fwd: null pointer");
  NSA_REQUIRE(p->K % 8 == 0 && p->K > 0, NSA_ERR_UNSUPPORTED_SHAPE, "act_fwd: K=%d must be a multiple of 8", p->K);
  NSA_REQUIRE(p->kind == 0 || p->kind == 1, NSA_ERR_BAD_ARG, "act_fwd: kind=%d", p->kind);
  int64_t n = p->M * (p->K / 8);
  if (n == 0) return NSA_OK;
  act_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("act_fwd");
}

extern "C" int nsa_act_bwd(const NsaActParams* p, void* stream) {
  NSA_REQUIRE(p && p->x && p->dy && p->dx, NSA_ERR_BAD_ARG, "act_bwd: null pointer");
  NSA_REQUIRE(p->K % 8 == 0 && p->K > 0, NSA_ERR_UNSUPPORTED_SHAPE, "act_bwd: K=%d must be a multiple of 8", p->K);
  NSA_REQUIRE(p->kind == 0 || p->kind == 1, NSA_ERR_BAD_ARG, "act_bwd: kind=%d", p->kind);
  int64_t n = p->M * (p->K / 8);
  if (n == 0) return NSA_OK;
  act_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("act_bwd");
}

extern "C" int nsa_combine_fwd(const NsaCombineParams* p, void* stream) {
  NSA_REQUIRE(p && p->a && p->b && p->c && p->w && p->y, NSA_ERR_BAD_ARG, "combine_fwd: null pointer");
  NSA_REQUIRE(p->D == 64 || p->D == 128 || p->D == 256, NSA_ERR_UNSUPPORTED_SHAPE, "combine_fwd: D=%d (64/128/256)", p->D);
  int64_t n = p->T * p->H * (p->D / 8);
  if (n == 0) return NSA_OK;
  combine_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("combine_fwd");
}

extern "C" int nsa_combine_bwd(const NsaCombineParams* p, void* stream) {
  NSA_REQUIRE(p && p->a && p->b && p->c && p->w && p->dy && p->da && p->db && p->dc && p->dw, NSA_ERR_BAD_ARG,
              "combine_bwd: null pointer");
  NSA_REQUIRE(p->D == 64 || p->D == 128 || p->D == 256, NSA_ERR_UNSUPPORTED_SHAPE, "combine_bwd: D=%d (64/128/256)", p->D);
  NSA_REQUIRE((!p->delta_a && !p->delta_b && !p->delta_c) || (p->delta_a && p->delta_b && p->delta_c), NSA_ERR_BAD_ARG,
              "combine_bwd: give all three delta outputs or none");
  int64_t n = p->T * p->H * (p->D / 8);
  if (n == 0) return NSA_OK;
  combine_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("combine_bwd");
}

extern "C" int nsa_store_kvcache(const NsaStoreKvParams* p, void* stream) {
  NSA_REQUIRE(p && p->key && p->value && p->k_cache && p->v_cache && p->slot_mapping, NSA_ERR_BAD_ARG, "store_kvcache: null pointer");
  NSA_REQUIRE(p->row_elems > 0 && p->row_elems % 8 == 0 && p->key_stride % 8 == 0 && p->value_stride % 8 == 0, NSA_ERR_BAD_ARG,
              "store_kvcache: rows must be multiples of 8 elements");
  const int64_t n = (int64_t)p->N * (p->row_elems / 8);
  if (n <= 0) return NSA_OK;
  store_kvcache_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("store_kvcache");
}

extern "C" int nsa_rope(const NsaRopeParams* p, void* stream) {
  NSA_REQUIRE(p && p->q && p->k && p->qe && p->ke && p->cos && p->sin, NSA_ERR_BAD_ARG, "rope: null pointer");
  NSA_REQUIRE(p->D > 0 && p->D % 16 == 0, NSA_ERR_UNSUPPORTED_SHAPE, "rope: D=%d must be a multiple of 16", p->D);
  NSA_REQUIRE((p->q_stride_h | p->q_stride_n | p->q_stride_b | p->k_stride_h | p->k_stride_n | p->k_stride_b | p->qe_stride_h |
               p->qe_stride_n | p->qe_stride_b | p->ke_stride_h | p->ke_stride_n | p->ke_stride_b | p->cos_stride_b | p->cos_stride_n) % 8 == 0,
              NSA_ERR_BAD_ARG, "rope: strides must be multiples of 8 elements (16-byte vectors)");
  NSA_REQUIRE(((uintptr_t)p->q | (uintptr_t)p->k | (uintptr_t)p->qe | (uintptr_t)p->ke | (uintptr_t)p->cos | (uintptr_t)p->sin) % 16 == 0,
              NSA_ERR_BAD_ARG, "rope: pointers must be 16-byte aligned");
  const int64_t n = (int64_t)p->B * p->N * (p->QH + p->KH) * (p->D / 16);
  if (n <= 0) return NSA_OK;
  rope_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("rope");
}

extern "C" int nsa_reorder(const NsaReorderParams* p, void* stream) {
  NSA_REQUIRE(p && p->x && p->y && p->x != p->y, NSA_ERR_BAD_ARG, "reorder: null or aliased pointer");
  NSA_REQUIRE(p->chunk_bytes % 16 == 0 && p->world_size > 0, NSA_ERR_BAD_ARG, "reorder: chunk_bytes %% 16 != 0");
  int64_t n = p->chunk_bytes / 16 * 2 * p->world_size;
  if (n == 0) return NSA_OK;
  reorder_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("reorder");
}

namespace nsa {
// rows [len_b, next multiple of 128) of every sequence's paged rows are cleared in both caches: the TMA-fed kernels read
// whole 128-row tiles, and rows past a sequence's end (never-written memory of its last page) must be finite
__global__ void paged_zero_tails_kernel(NsaPagedPoolParams p) {
  const int b = blockIdx.x;
  int len = p.context_lens[b];
  if (p.decode == 2) len = len >= p.kernel_size ? (len - p.kernel_size) / p.stride + 1 : 0;   // compressed rows of the context
  if (len <= 0) return;
  const int end = min((len + 127) / 128 * 128, p.table_stride * p.page_size);
  const int sh = 31 - __clz(p.page_size);
  const int chunks = (int)(p.row_stride / 8);   // 16-byte pieces of one cache row (all heads)
  const int32_t* tab = p.kv_table + (int64_t)b * p.table_stride;
  for (int i = threadIdx.x; i < (end - len) * chunks; i += blockDim.x) {
    const int r = len + i / chunks, c = i % chunks;
    const int page = tab[r >> sh];
    if (page < 0) continue;
    const int64_t off = (((int64_t)page << sh) + (r & (p.page_size - 1))) * p.row_stride + c * 8;
    reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.cache0) + off)[0] = make_uint4(0, 0, 0, 0);
    if (p.cache1) reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.cache1) + off)[0] = make_uint4(0, 0, 0, 0);
  }
}
}  // namespace nsa

namespace nsa {
// dst[y_cu[b] + j] = cache[row of (b, j) in the page table], all heads of a row, for j < y_cu[b+1] - y_cu[b]
__global__ void paged_gather_rows_kernel(NsaPagedPoolParams p) {
  const int b = blockIdx.y;
  const int y0 = p.y_cu[b], n = p.y_cu[b + 1] - y0;
  const int sh = 31 - __clz(p.page_size);
  const int chunks = (int)(p.row_stride / 8);
  const int32_t* tab = p.kv_table + (int64_t)b * p.table_stride;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n * chunks; i += gridDim.x * blockDim.x) {
    const int j = i / chunks, c = i - j * chunks;
    const int64_t src = (((int64_t)tab[j >> sh] << sh) + (j & (p.page_size - 1))) * p.row_stride + c * 8;
    reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.cache1) + ((int64_t)y0 + j) * p.row_stride + c * 8)[0] =
        *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.cache0) + src);
  }
}
}  // namespace nsa

extern "C" int nsa_paged_gather_rows(const NsaPagedPoolParams* p, void* stream) {
  NSA_REQUIRE(p && p->cache0 && p->cache1 && p->kv_table && p->y_cu, NSA_ERR_BAD_ARG, "paged_gather_rows: null pointer");
  NSA_REQUIRE(p->page_size > 0 && (p->page_size & (p->page_size - 1)) == 0 && p->row_stride % 8 == 0, NSA_ERR_UNSUPPORTED_SHAPE,
              "paged_gather_rows: page=%d must be a power of two and rows multiples of 16 bytes", p->page_size);
  if (p->B <= 0 || p->y_maxlen <= 0) return NSA_OK;
  const int64_t work = (int64_t)p->y_maxlen * (p->row_stride / 8);
  dim3 grid((unsigned)std::min<int64_t>((work + 255) / 256, 1024), p->B);
  paged_gather_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("paged_gather_rows");
}

extern "C" int nsa_paged_zero_tails(const NsaPagedPoolParams* p, void* stream) {
  NSA_REQUIRE(p && p->cache0 && p->kv_table && p->context_lens, NSA_ERR_BAD_ARG, "paged_zero_tails: null pointer");
  NSA_REQUIRE(p->page_size > 0 && (p->page_size & (p->page_size - 1)) == 0 && p->row_stride % 8 == 0, NSA_ERR_UNSUPPORTED_SHAPE,
              "paged_zero_tails: page=%d must be a power of two and rows multiples of 16 bytes", p->page_size);
  NSA_REQUIRE(p->decode != 2 || (p->kernel_size > 0 && p->stride > 0), NSA_ERR_BAD_ARG, "paged_zero_tails: kernel_size / stride");
  if (p->B <= 0) return NSA_OK;
  paged_zero_tails_kernel<<<p->B, 256, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("paged_zero_tails");
}

extern "C" int nsa_paged_mean_pool(const NsaPagedPoolParams* p, void* stream) {
  NSA_REQUIRE(p && p->cache0 && p->slot_mapping && p->kv_table, NSA_ERR_BAD_ARG, "paged_mean_pool: null pointer");
  NSA_REQUIRE(p->decode ? p->context_lens != nullptr : p->y_cu != nullptr, NSA_ERR_BAD_ARG, "paged_mean_pool: missing length table");
  NSA_REQUIRE(p->D % 8 == 0 && p->D > 0 && p->page_size > 0, NSA_ERR_UNSUPPORTED_SHAPE, "paged_mean_pool: D=%d page=%d", p->D, p->page_size);
  if (p->B <= 0) return NSA_OK;
  int rows = p->decode ? 1 : p->y_maxlen;
  if (rows <= 0) return NSA_OK;
  const int CH = p->D / 8;
  dim3 grid((unsigned)(((int64_t)rows * CH + 63) / 64), p->B, p->H * (p->cache1 ? 2 : 1));
  paged_pool_kernel<<<grid, 64, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("paged_mean_pool");
}
