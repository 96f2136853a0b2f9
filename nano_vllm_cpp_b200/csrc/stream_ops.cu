// Several copies of the residual stream ("streams"), the norm without statistics that reads them, and the scaling
// and soft cap of the logits.
//
// stream_mix_norm: per row t the model keeps S copies x[t, 0..S-1, :] (float32).  One launch
//   1. brings the copies up to date with the sublayer output y[t, :] that is still pending:
//        x'[d] = sum_c carry[c, d] * x[c] + write[d] * y          (all d at once from the old copies)
//      where y is a dense float32 matrix or a weighted sum of rows that has not been taken yet
//        y[t, :] = dense[t, :] + sum_r weight[t, r] * rows[index[t, r], :]      (r in order, as add_rmsnorm takes it);
//      without carry and write the update is x'[d] = x[d] + y (one copy: the usual residual sum);
//   2. reads them for the next sublayer:  u = sum_d read[d] * x'[d]   (read == nullptr: the plain sum of the copies);
//   3. norms u:  kind 1, "dynamic tanh":  tanh(alpha * u) * gain + shift, with no mean and no variance, so that
//      nothing is reduced over the row and a thread needs only its own columns; kind 0: u itself;
//   4. writes the result in the activation dtype and/or in float32.
// Everything is float32 arithmetic.  A thread owns VEC neighbouring columns of one row and keeps the S copies of
// them in registers, so the update is safe in place.
#include "common.cuh"

namespace {

constexpr int SM_MAX_STREAMS = 8, SM_MAX_R = 64, SM_THREADS = 256;

struct StreamArgs {
  float* x;                 // [T, S, H]
  const float* branch;      // [T, H] or nullptr
  const float* rows;        // the mix: [*, H]
  const int* index;         // [T, R]
  const float* weight;      // [T, R]
  const float* dense;       // [T, H] or nullptr
  const float* carry;       // [S, S] (from, to) or nullptr
  const float* write;       // [S] or nullptr
  const float* read;        // [S] or nullptr
  const float* alpha;       // one float
  const float* gain;        // [H]
  const float* shift;       // [H]
  void* out;                // [T, H] in out_dt, or nullptr
  float* out32;             // [T, H] or nullptr
  int out_dt, H, S, R, kind, update;
};

template <int VEC>
struct Cols { float v[VEC]; };

template <int VEC>
__device__ __forceinline__ Cols<VEC> ld_cols(const float* p) {
  Cols<VEC> c;
  if (VEC == 4) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    c.v[0] = q.x; c.v[VEC > 1 ? 1 : 0] = q.y; c.v[VEC > 2 ? 2 : 0] = q.z; c.v[VEC > 3 ? 3 : 0] = q.w;
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) c.v[j] = p[j];
  }
  return c;
}
template <int VEC>
__device__ __forceinline__ void st_cols(float* p, const Cols<VEC>& c) {
  if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(c.v[0], c.v[VEC > 1 ? 1 : 0], c.v[VEC > 2 ? 2 : 0], c.v[VEC > 3 ? 3 : 0]);
  else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) p[j] = c.v[j];
  }
}

// SMAX: the most copies this instance keeps in registers (1, 2, 4 or 8): a thread's registers, and with them how many
// blocks share a multiprocessor, follow the model's number of copies and not the largest number allowed.
template <int VEC, int SMAX>
__global__ void __launch_bounds__(SM_THREADS) stream_mix_norm_kernel(StreamArgs a) {
  __shared__ float s_carry[SM_MAX_STREAMS * SM_MAX_STREAMS], s_write[SM_MAX_STREAMS], s_read[SM_MAX_STREAMS];
  __shared__ int s_idx[SM_MAX_R];
  __shared__ float s_w[SM_MAX_R];
  const int t = blockIdx.x, tid = threadIdx.x, S = a.S;
  grid_dep_wait();
  grid_dep_launch();
  for (int i = tid; i < S * S; i += blockDim.x) s_carry[i] = a.carry ? a.carry[i] : (i / S == i % S ? 1.f : 0.f);
  for (int i = tid; i < S; i += blockDim.x) {
    s_write[i] = a.write ? a.write[i] : 1.f;
    s_read[i] = a.read ? a.read[i] : 1.f;
  }
  for (int i = tid; i < a.R; i += blockDim.x) {
    s_idx[i] = a.index[(size_t)t * a.R + i];
    s_w[i] = a.weight[(size_t)t * a.R + i];
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + tid;      // this thread's chunk of columns
  if (c * VEC >= a.H) return;
  const size_t col = (size_t)c * VEC;
  float* xr = a.x + (size_t)t * S * a.H + col;
  Cols<VEC> xs[SMAX];
#pragma unroll
  for (int s = 0; s < SMAX; ++s)
    if (s < S) xs[s] = ld_cols<VEC>(xr + (size_t)s * a.H);
  if (a.update) {
    Cols<VEC> y;
    if (a.branch) {
      y = ld_cols<VEC>(a.branch + (size_t)t * a.H + col);
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) y.v[j] = 0.f;
      int k = 0;
      for (; k + 4 <= a.R; k += 4) {          // four rows' loads in flight; the sum keeps the order of k
        Cols<VEC> r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) r[u] = ld_cols<VEC>(a.rows + (size_t)s_idx[k + u] * a.H + col);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int j = 0; j < VEC; ++j) y.v[j] = fmaf(s_w[k + u], r[u].v[j], y.v[j]);
      }
      for (; k < a.R; ++k) {
        const Cols<VEC> r = ld_cols<VEC>(a.rows + (size_t)s_idx[k] * a.H + col);
#pragma unroll
        for (int j = 0; j < VEC; ++j) y.v[j] = fmaf(s_w[k], r.v[j], y.v[j]);
      }
      if (a.dense) {
        const Cols<VEC> d = ld_cols<VEC>(a.dense + (size_t)t * a.H + col);
#pragma unroll
        for (int j = 0; j < VEC; ++j) y.v[j] += d.v[j];
      }
    }
    Cols<VEC> nx[SMAX];
#pragma unroll
    for (int d = 0; d < SMAX; ++d) {
      if (d < S) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) nx[d].v[j] = s_write[d] * y.v[j];
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < S) {
            const float m = s_carry[s * S + d];
#pragma unroll
            for (int j = 0; j < VEC; ++j) nx[d].v[j] = fmaf(m, xs[s].v[j], nx[d].v[j]);
          }
      }
    }
#pragma unroll
    for (int d = 0; d < SMAX; ++d)
      if (d < S) {
        xs[d] = nx[d];
        st_cols<VEC>(xr + (size_t)d * a.H, xs[d]);
      }
  }
  if (!a.out && !a.out32) return;
  Cols<VEC> u;
#pragma unroll
  for (int j = 0; j < VEC; ++j) u.v[j] = 0.f;
#pragma unroll
  for (int s = 0; s < SMAX; ++s)
    if (s < S) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) u.v[j] = fmaf(s_read[s], xs[s].v[j], u.v[j]);
    }
  if (a.kind == 1) {
    const float al = a.alpha[0];
    const Cols<VEC> g = ld_cols<VEC>(a.gain + col), b = ld_cols<VEC>(a.shift + col);
#pragma unroll
    for (int j = 0; j < VEC; ++j) u.v[j] = fmaf(tanhf(al * u.v[j]), g.v[j], b.v[j]);
  }
  if (a.out32) st_cols<VEC>(a.out32 + (size_t)t * a.H + col, u);
  if (a.out) {
    if (a.out_dt == NV_DT_F32) st_cols<VEC>((float*)a.out + (size_t)t * a.H + col, u);
    else {
      bf16* o = (bf16*)a.out + (size_t)t * a.H + col;
      if (VEC == 4) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(u.v[0], u.v[VEC > 1 ? 1 : 0]),
                             hi = __floats2bfloat162_rn(u.v[VEC > 2 ? 2 : 0], u.v[VEC > 3 ? 3 : 0]);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(o) = pk;
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) o[j] = __float2bfloat16_rn(u.v[j]);
      }
    }
  }
}

// z = cap * tanh(scale * z / cap), or scale * z without a cap; float32, in place.
__global__ void scale_softcap_kernel(float* __restrict__ z, long long n, float scale, float cap) {
  grid_dep_wait();
  grid_dep_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = z[i] * scale;
  z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

}  // namespace

NV_API int nv_stream_mix_norm_limits(int what) { return what == 0 ? SM_MAX_STREAMS : SM_MAX_R; }

NV_API int nv_stream_mix_norm(float* x, int T, int S, int H, const float* branch, const float* rows, const int* index,
                              const float* weight, int R, const float* dense, const float* carry, const float* write,
                              const float* read, int kind, const float* alpha, const float* gain, const float* shift,
                              void* out, int out_dt, float* out32, cudaStream_t s) {
  if (out && !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (S < 1 || S > SM_MAX_STREAMS || H < 1 || R < 0 || R > SM_MAX_R) return NV_ERR_BAD_SIZE;
  if (R > 0 && (!rows || !index || !weight)) return NV_ERR_BAD_SIZE;
  if (branch && (R > 0 || dense)) return NV_ERR_BAD_SIZE;          // one form of the pending output at a time
  if ((carry == nullptr) != (write == nullptr)) return NV_ERR_BAD_SIZE;
  if (!carry && S != 1 && (branch || R > 0 || dense)) return NV_ERR_BAD_SIZE;
  if (kind < 0 || kind > 1 || (kind == 1 && (!alpha || !gain || !shift))) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  StreamArgs a;
  a.x = x; a.branch = branch; a.rows = rows; a.index = index; a.weight = weight; a.dense = dense; a.carry = carry;
  a.write = write; a.read = read; a.alpha = alpha; a.gain = gain; a.shift = shift; a.out = out; a.out32 = out32;
  a.out_dt = out_dt; a.H = H; a.S = S; a.R = R; a.kind = kind;
  a.update = (branch || R > 0 || dense) ? 1 : 0;
  const int vec = H % 4 == 0 ? 4 : 1;
  const int chunks = H / vec;
  int threads = 32;
  while (threads < SM_THREADS && threads < chunks) threads *= 2;
  const dim3 grid((unsigned)T, (unsigned)((chunks + threads - 1) / threads));
#define NV_STREAM_LAUNCH(SMAX)                                                                              \
  do {                                                                                                      \
    if (vec == 4) NV_RETURN_IF(launch_dep(stream_mix_norm_kernel<4, SMAX>, grid, dim3(threads), 0, s, a)); \
    else NV_RETURN_IF(launch_dep(stream_mix_norm_kernel<1, SMAX>, grid, dim3(threads), 0, s, a));          \
  } while (0)
  if (S == 1) NV_STREAM_LAUNCH(1);
  else if (S == 2) NV_STREAM_LAUNCH(2);
  else if (S <= 4) NV_STREAM_LAUNCH(4);
  else NV_STREAM_LAUNCH(8);
#undef NV_STREAM_LAUNCH
  NV_RETURN_LAST();
}

NV_API int nv_scale_softcap(float* z, long long n, float scale, float cap, cudaStream_t s) {
  if (n <= 0) return NV_OK;
  NV_RETURN_IF(launch_dep(scale_softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, z, n, scale, cap));
  NV_RETURN_LAST();
}
