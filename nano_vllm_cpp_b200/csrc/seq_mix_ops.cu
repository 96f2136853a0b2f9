// Kernels of the mixers that keep a fixed-size state per request, and of the layer pieces around them:
//
//   branch_norm_add   x += rms(y) * w, y one branch or the mean of several RMS-normed, weighted branches;
//                     also the residual stream's rows in the activation type for the products that read them
//   activation        gelu (erf or tanh form) or silu over a matrix
//   token_gate        gelu_tanh(gate) * table[token, columns of this layer]
//   conv_silu_norm    short causal convolution per channel over time with silu; q and k heads made unit vectors
//   conv_state_update the last taps - 1 inputs of every channel, kept per request
//   mlstm_scan        matrix memory with exponential input gate, a running maximum and a normaliser state
//   gated_delta_scan  matrix memory with a decay per head and the delta rule
//   qk_prepare_store  q/k head norm, rotation of pairs (interleaved or split halves), keys and values to their pages
//   paged_attention_general   softmax attention over paged keys with separate key and value sizes and an optional sink
//
// Everything that enters a recurrence, every norm, every gate, angle, score and weight is computed in 32-bit floats
// whatever the storage type of the activations is.  The sums of a row are taken in an order that depends on the
// row alone (its own block, a thread's elements in order, a fixed tree over threads), so a row's result does not
// depend on what else is in the batch nor on how its sequence was cut into steps.
#include "common.cuh"

#include <algorithm>

namespace {

constexpr int SM_THREADS = 256;

// Sum over the block, the same order for every call; `red` holds blockDim.x / 32 floats.  All threads get the sum.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();          // (red may still be read from the call before)
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nw; ++i) s += red[i];
  return s;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float gelu_erf_(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f)); }
__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------ branch norm + residual sum
constexpr int MAX_BRANCHES = 4;
struct BranchArgs {
  float* x;                         // [T, H] residual stream, updated in place
  const float* br[MAX_BRANCHES];    // [T, H] branch outputs
  const float* bw[MAX_BRANCHES];    // [H] weights of the branches' own norms (all given, or none with nb == 1)
  const float* w;                   // [H] weight of the norm over the (mixed) branch
  void* out;                        // [T, H] x after the sum, in out_dt (may be null)
  int nb, H, out_dt;
  float eps, mix_scale;
};

__global__ void __launch_bounds__(SM_THREADS) branch_norm_add_kernel(BranchArgs a) {
  extern __shared__ float ysm[];    // H floats
  __shared__ float red[SM_THREADS / 32];
  const int t = blockIdx.x, tid = threadIdx.x, H = a.H;
  const size_t base = (size_t)t * H;
  if (a.nb == 0) {
    if (a.out)
      for (int i = tid; i < H; i += SM_THREADS) st_dt(a.out, a.out_dt, base + i, a.x[base + i]);
    return;
  }
  if (a.bw[0]) {
    for (int i = tid; i < H; i += SM_THREADS) ysm[i] = 0.f;
    for (int b = 0; b < a.nb; ++b) {
      float ss = 0.f;
      for (int i = tid; i < H; i += SM_THREADS) { float v = a.br[b][base + i]; ss = fmaf(v, v, ss); }
      const float r = rsqrtf(block_sum(ss, red) / (float)H + a.eps);
      for (int i = tid; i < H; i += SM_THREADS) ysm[i] += a.br[b][base + i] * r * a.bw[b][i];
    }
    for (int i = tid; i < H; i += SM_THREADS) ysm[i] *= a.mix_scale;
  } else {
    for (int i = tid; i < H; i += SM_THREADS) ysm[i] = a.br[0][base + i];
  }
  float ss = 0.f;
  for (int i = tid; i < H; i += SM_THREADS) ss = fmaf(ysm[i], ysm[i], ss);
  const float r = rsqrtf(block_sum(ss, red) / (float)H + a.eps);
  for (int i = tid; i < H; i += SM_THREADS) {
    const float v = a.x[base + i] + ysm[i] * r * a.w[i];
    a.x[base + i] = v;
    if (a.out) st_dt(a.out, a.out_dt, base + i, v);
  }
}

// ------------------------------------------------------------------ activation over a matrix
__global__ void activation_kernel(const void* __restrict__ in, int in_dt, void* __restrict__ out, int out_dt,
                                  long long n, int kind) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float z = ld_dt(in, in_dt, i);
  st_dt(out, out_dt, i, kind == 0 ? gelu_erf_(z) : (kind == 1 ? gelu_tanh_(z) : siluf_(z)));
}

// ------------------------------------------------------------------ gate times a per-token table row
// out[t, j] = gelu_tanh(gate[t, j]) * table[id(t), col0 + j]; a negative id -(r + 1) is read from feed[r]
__global__ void token_gate_kernel(const void* __restrict__ gate, int gate_dt, long long gate_ld,
                                  const int* __restrict__ ids, const int* __restrict__ feed,
                                  const void* __restrict__ table, int table_dt, long long table_ld, int col0, int d,
                                  int V, void* __restrict__ out, int out_dt, int* __restrict__ err) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && feed) id = feed[-id - 1];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicExch(err, 1 + t);
    id = 0;
  }
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    const float g = gelu_tanh_(ld_dt(gate, gate_dt, (size_t)t * gate_ld + j));
    st_dt(out, out_dt, (size_t)t * d + j, g * ld_dt(table, table_dt, (size_t)id * table_ld + col0 + j));
  }
}

// ------------------------------------------------------------------ short convolution over time
// in: [T, ld] float32 or bfloat16, channels col0 .. col0 + C; w: [C, taps] float32, the last column the current token's;
// state: per slot [taps - 1, C] float32, the inputs of the request's last taps - 1 positions (zero before its start).
// out[t, c] = silu(sum_d w[c, taps - 1 - d] * in(t - d)); then every one of the first `unit_heads` heads of
// `unit_dim` channels is divided by sqrt(sum of squares + unit_eps), and the first `scaled_heads` of them also
// multiplied by `scale`.  One block per row.
__global__ void __launch_bounds__(SM_THREADS) conv_silu_norm_kernel(
    const void* __restrict__ in, int in_dt, long long ld, int col0, int C, const float* __restrict__ w, int taps,
    const int* __restrict__ row_entry, const int* __restrict__ cu_rows, const int* __restrict__ entry_slot,
    const float* __restrict__ state, long long slot_stride, int unit_heads, int unit_dim, float unit_eps,
    int scaled_heads, float scale, float* __restrict__ out) {
  extern __shared__ float ysm[];    // C floats
  const int t = blockIdx.x, tid = threadIdx.x;
  const int e = row_entry[t];
  const int j = t - cu_rows[e];
  const float* st = state + (size_t)entry_slot[e] * slot_stride;
  for (int c = tid; c < C; c += SM_THREADS) {
    float acc = 0.f;
    for (int d = 0; d < taps; ++d) {
      const int jj = j - d;
      const float v = jj >= 0 ? ld_dt(in, in_dt, (size_t)(t - d) * ld + col0 + c) : st[(size_t)(taps - 1 + jj) * C + c];
      acc = fmaf(w[(size_t)c * taps + (taps - 1 - d)], v, acc);
    }
    ysm[c] = siluf_(acc);
  }
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5;
  for (int h = warp; h < unit_heads; h += SM_THREADS / 32) {
    float ss = 0.f;
    for (int i = lane; i < unit_dim; i += 32) { float v = ysm[h * unit_dim + i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss + unit_eps) * (h < scaled_heads ? scale : 1.f);
    for (int i = lane; i < unit_dim; i += 32) ysm[h * unit_dim + i] *= r;
  }
  __syncthreads();
  for (int c = tid; c < C; c += SM_THREADS) out[(size_t)t * C + c] = ysm[c];
}

// After the convolution has read the old state: state[s] = the input at the entry's position end - (taps - 1) + s.
// A thread owns a channel and goes through s upward, so what it still has to read (old[s + len]) lies above what
// it has written.
__global__ void conv_state_update_kernel(const void* __restrict__ in, int in_dt, long long ld, int col0, int C,
                                         int taps, const int* __restrict__ cu_rows,
                                         const int* __restrict__ entry_slot, float* __restrict__ state,
                                         long long slot_stride) {
  const int e = blockIdx.x;
  const int row0 = cu_rows[e], len = cu_rows[e + 1] - row0;
  float* st = state + (size_t)entry_slot[e] * slot_stride;
  for (int c = threadIdx.x; c < C; c += blockDim.x)
    for (int s = 0; s < taps - 1; ++s) {
      const int jj = len - (taps - 1) + s;
      st[(size_t)s * C + c] = jj >= 0 ? ld_dt(in, in_dt, (size_t)(row0 + jj) * ld + col0 + c) : st[(size_t)(s + len) * C + c];
    }
}

// ------------------------------------------------------------------ matrix memories, token by token
// One block per (entry, head).  The head's matrix S [dk, dv] lives in shared memory while the entry's rows run and
// goes back to the request's state afterwards.  Thread (c, rs) = (tid % dv, tid / dv) owns column c and the rows
// r = rs, rs + RS, ...; sums over rows are taken per thread in that order and then over rs in order.
struct ScanCommon {
  const int* cu_rows;
  const int* entry_slot;
  float* S;                 // [slots][H, dk, dv]
  long long S_stride;
  const float* norm_w;
  void* out;                // [T, H * dv]
  int out_dt, H, dk, dv;
  float eps;
};

struct MlstmArgs {
  ScanCommon c;
  const float* proj;        // [T, ld] float32: q | k | v | gate | i | f at their columns
  long long ld;
  int q0, k0, v0, g0, i0, f0;
  float* n;                 // [slots][H, dk]
  long long n_stride;
  float* m;                 // [slots][H]
  long long m_stride;
  float cap, q_scale, den_eps;
  int norm_per_head;        // the norm weight has H * dv entries (else dv, shared by the heads)
};

__global__ void __launch_bounds__(SM_THREADS) mlstm_scan_kernel(MlstmArgs a) {
  extern __shared__ float sm[];
  const int dk = a.c.dk, dv = a.c.dv, H = a.c.H;
  const int RS = max(1, min(SM_THREADS / dv, dk));
  float* S = sm;                     // dk * dv
  float* nn = S + dk * dv;           // dk
  float* q = nn + dk;                // dk
  float* k = q + dk;                 // dk
  float* v = k + dk;                 // dv
  float* part = v + dv;              // RS * dv
  float* o = part + RS * dv;         // dv
  float* sc = o + dv;                // 8 scalars
  const int e = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int row0 = a.c.cu_rows[e], row1 = a.c.cu_rows[e + 1];
  const int slot = a.c.entry_slot[e];
  float* Sg = a.c.S + (size_t)slot * a.c.S_stride + (size_t)h * dk * dv;
  float* ng = a.n + (size_t)slot * a.n_stride + (size_t)h * dk;
  float* mg = a.m + (size_t)slot * a.m_stride + h;
  for (int i = tid; i < dk * dv; i += SM_THREADS) S[i] = Sg[i];
  for (int i = tid; i < dk; i += SM_THREADS) nn[i] = ng[i];
  float m = *mg;
  const int c = tid % dv, rs = tid / dv;
  const bool owner = tid < RS * dv;
  __syncthreads();
  for (int t = row0; t < row1; ++t) {
    const float* p = a.proj + (size_t)t * a.ld;
    for (int i = tid; i < dk; i += SM_THREADS) {
      q[i] = p[a.q0 + h * dk + i] * a.q_scale;
      k[i] = p[a.k0 + h * dk + i];
    }
    for (int i = tid; i < dv; i += SM_THREADS) v[i] = p[a.v0 + h * dv + i];
    // gates: every thread computes the same numbers
    const float ig = a.cap * tanhf(p[a.i0 + h] / a.cap);
    const float fg = logsigmoidf_(a.cap * tanhf(p[a.f0 + h] / a.cap));
    const float m_new = fmaxf(fg + m, ig);
    const float fa = expf(fg + m - m_new), ib = expf(ig - m_new);
    m = m_new;
    __syncthreads();
    if (tid < 32) {                  // the normaliser state and its product with q
      float acc = 0.f;
      for (int r = tid; r < dk; r += 32) {
        const float x = fa * nn[r] + ib * k[r];
        nn[r] = x;
        acc = fmaf(x, q[r], acc);
      }
      acc = warp_sum(acc);
      if (tid == 0) sc[0] = acc;
    }
    if (owner) {
      float acc = 0.f;
      const float bv = ib * v[c];
      for (int r = rs; r < dk; r += RS) {
        const float s = fa * S[r * dv + c] + k[r] * bv;
        S[r * dv + c] = s;
        acc = fmaf(s, q[r], acc);
      }
      part[rs * dv + c] = acc;
    }
    __syncthreads();
    if (tid < dv) {
      float num = 0.f;
      for (int i = 0; i < RS; ++i) num += part[i * dv + tid];
      const float den = fmaxf(fabsf(sc[0]), expf(-m)) + a.den_eps;
      o[tid] = num / den;
    }
    __syncthreads();
    if (tid < 32) {
      float ss = 0.f;
      for (int i = tid; i < dv; i += 32) ss = fmaf(o[i], o[i], ss);
      ss = warp_sum(ss);
      if (tid == 0) sc[1] = rsqrtf(ss / (float)dv + a.c.eps);
    }
    __syncthreads();
    if (tid < dv) {
      const float w = a.c.norm_w[a.norm_per_head ? h * dv + tid : tid];
      const float gate = sigmoidf_(p[a.g0 + h * dv + tid]);
      st_dt(a.c.out, a.c.out_dt, (size_t)t * H * dv + (size_t)h * dv + tid, o[tid] * sc[1] * w * gate);
    }
  }
  __syncthreads();
  for (int i = tid; i < dk * dv; i += SM_THREADS) Sg[i] = S[i];
  for (int i = tid; i < dk; i += SM_THREADS) ng[i] = nn[i];
  if (tid == 0) *mg = m;
}

struct DeltaArgs {
  ScanCommon c;
  const float* qkv;         // [T, C] float32 after convolution, activation and unit norm: q | k | v
  int C, q0, k0, v0, G;     // G heads of q and k; head h reads q/k head h / (H / G)
  const void* proj;         // [T, ld]: output gate, beta and decay pre-activations at their columns
  int proj_dt;
  long long ld;
  int g0, b0, a0;
  const float* A_log;       // [H]
  const float* dt_bias;     // [H]
};

__global__ void __launch_bounds__(SM_THREADS) gated_delta_scan_kernel(DeltaArgs a) {
  extern __shared__ float sm[];
  const int dk = a.c.dk, dv = a.c.dv, H = a.c.H;
  const int RS = max(1, min(SM_THREADS / dv, dk));
  float* S = sm;                     // dk * dv
  float* q = S + dk * dv;            // dk
  float* k = q + dk;                 // dk
  float* v = k + dk;                 // dv
  float* partk = v + dv;             // RS * dv
  float* partq = partk + RS * dv;    // RS * dv
  float* u = partq + RS * dv;        // dv
  float* o = u + dv;                 // dv
  float* sc = o + dv;                // 8 scalars
  const int e = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int gh = h / (H / a.G);
  const int row0 = a.c.cu_rows[e], row1 = a.c.cu_rows[e + 1];
  float* Sg = a.c.S + (size_t)a.c.entry_slot[e] * a.c.S_stride + (size_t)h * dk * dv;
  for (int i = tid; i < dk * dv; i += SM_THREADS) S[i] = Sg[i];
  const int c = tid % dv, rs = tid / dv;
  const bool owner = tid < RS * dv;
  const float rate = expf(a.A_log[h]), dtb = a.dt_bias[h];
  __syncthreads();
  for (int t = row0; t < row1; ++t) {
    const float* x = a.qkv + (size_t)t * a.C;
    for (int i = tid; i < dk; i += SM_THREADS) {
      q[i] = x[a.q0 + gh * dk + i];
      k[i] = x[a.k0 + gh * dk + i];
    }
    for (int i = tid; i < dv; i += SM_THREADS) v[i] = x[a.v0 + h * dv + i];
    const float beta = sigmoidf_(ld_dt(a.proj, a.proj_dt, (size_t)t * a.ld + a.b0 + h));
    const float g = expf(-rate * softplusf_(ld_dt(a.proj, a.proj_dt, (size_t)t * a.ld + a.a0 + h) + dtb));
    __syncthreads();
    if (tid < 32) {
      float acc = 0.f;
      for (int r = tid; r < dk; r += 32) acc = fmaf(k[r], q[r], acc);
      acc = warp_sum(acc);
      if (tid == 0) sc[0] = acc;
    }
    if (owner) {
      float ak = 0.f, aq = 0.f;
      for (int r = rs; r < dk; r += RS) {
        const float s = S[r * dv + c];
        ak = fmaf(s, k[r], ak);
        aq = fmaf(s, q[r], aq);
      }
      partk[rs * dv + c] = ak;
      partq[rs * dv + c] = aq;
    }
    __syncthreads();
    if (tid < dv) {
      float sk = 0.f, sq = 0.f;
      for (int i = 0; i < RS; ++i) { sk += partk[i * dv + tid]; sq += partq[i * dv + tid]; }
      const float uu = beta * (v[tid] - g * sk);
      u[tid] = uu;
      o[tid] = g * sq + sc[0] * uu;
    }
    __syncthreads();
    if (owner) {
      const float uu = u[c];
      for (int r = rs; r < dk; r += RS) S[r * dv + c] = g * S[r * dv + c] + k[r] * uu;
    }
    if (tid < 32) {
      float ss = 0.f;
      for (int i = tid; i < dv; i += 32) ss = fmaf(o[i], o[i], ss);
      ss = warp_sum(ss);
      if (tid == 0) sc[1] = rsqrtf(ss / (float)dv + a.c.eps);
    }
    __syncthreads();
    if (tid < dv) {
      const float gate = siluf_(ld_dt(a.proj, a.proj_dt, (size_t)t * a.ld + a.g0 + h * dv + tid));
      st_dt(a.c.out, a.c.out_dt, (size_t)t * H * dv + (size_t)h * dv + tid, o[tid] * sc[1] * a.c.norm_w[tid] * gate);
    }
  }
  __syncthreads();
  for (int i = tid; i < dk * dv; i += SM_THREADS) Sg[i] = S[i];
}

// ------------------------------------------------------------------ q/k head norm, rotation, cache write
// in: [T, ld] with q at q0 (Hq * D), k at k0 (Hkv * D), v at v0 (Hkv * Dv).  Per q and k head: RMS norm over D with
// the weight qw / kw (null: no norm); then the first rot_dim elements are turned in pairs, (2i, 2i + 1) if
// `interleaved` else (i, i + rot_dim / 2), by the angle position * inv_freq[i], cosine and sine times `amplitude`.
// q goes to q_out [T, Hq * D]; k and v go to the row's place in their pages.  One block per row, a warp per head.
struct QkArgs {
  const void* in;
  int in_dt;
  long long ld;
  int q0, k0, v0;
  const int* positions;
  const int* row_entry;
  const int* block_table;
  int max_blocks;
  const float* qw;
  const float* kw;
  float eps;
  const float* inv_freq;
  int rot_dim, interleaved;
  float amplitude;
  void* q_out;
  int q_dt;
  void* kc;
  void* vc;
  int cache_dt;
  int Hq, Hkv, D, Dv, page, write_kv;
  int* err;
};

constexpr int QK_THREADS = 128;

__global__ void __launch_bounds__(QK_THREADS) qk_prepare_store_kernel(QkArgs a) {
  extern __shared__ float sm[];      // per warp D floats
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = a.D, half = a.rot_dim / 2;
  float* buf = sm + warp * D;
  const int pos = a.positions[t];
  int blk = 0, write_kv = a.write_kv;
  if (write_kv) {
    blk = a.block_table[(size_t)a.row_entry[t] * a.max_blocks + pos / a.page];
    if (blk < 0) {
      if (threadIdx.x == 0) atomicExch(a.err, 1 + t);
      write_kv = 0;
    }
  }
  const size_t slot = (size_t)(pos % a.page);
  const int heads = a.Hq + (write_kv ? a.Hkv : 0);
  for (int h = warp; h < heads; h += QK_THREADS / 32) {
    const bool is_q = h < a.Hq;
    const size_t src = (size_t)t * a.ld + (is_q ? a.q0 + h * D : a.k0 + (h - a.Hq) * D);
    const float* w = is_q ? a.qw : a.kw;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float x = ld_dt(a.in, a.in_dt, src + i);
      buf[i] = x;
      ss = fmaf(x, x, ss);
    }
    if (w) {
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)D + a.eps);
      for (int i = lane; i < D; i += 32) buf[i] = buf[i] * r * w[i];
    }
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
      const int i0 = a.interleaved ? 2 * i : i, i1 = a.interleaved ? 2 * i + 1 : i + half;
      const float ang = (float)pos * a.inv_freq[i];
      const float cs = cosf(ang) * a.amplitude, sn = sinf(ang) * a.amplitude;
      const float x0 = buf[i0], x1 = buf[i1];
      buf[i0] = x0 * cs - x1 * sn;
      buf[i1] = x1 * cs + x0 * sn;
    }
    __syncwarp();
    if (is_q) {
      for (int i = lane; i < D; i += 32) st_dt(a.q_out, a.q_dt, (size_t)t * a.Hq * D + (size_t)h * D + i, buf[i]);
    } else {
      const size_t dst = (((size_t)blk * a.Hkv + (h - a.Hq)) * a.page + slot) * D;
      for (int i = lane; i < D; i += 32) st_dt(a.kc, a.cache_dt, dst + i, buf[i]);
    }
    __syncwarp();
  }
  if (write_kv) {
    for (int i = threadIdx.x; i < a.Hkv * a.Dv; i += QK_THREADS) {
      const int hv = i / a.Dv, d = i % a.Dv;
      const size_t dst = (((size_t)blk * a.Hkv + hv) * a.page + slot) * a.Dv + d;
      st_dt(a.vc, a.cache_dt, dst, ld_dt(a.in, a.in_dt, (size_t)t * a.ld + a.v0 + i));
    }
  }
}

// ------------------------------------------------------------------ paged softmax attention, general sizes
// One block per (row, query head).  Keys of D elements, values of Dv; with `has_sink` the softmax's denominator
// also holds exp(sink_score): a key with that score and no value.  Chunks of ATTG_THREADS keys, running maximum.
constexpr int ATTG_THREADS = 128;

__global__ void __launch_bounds__(ATTG_THREADS) paged_attention_general_kernel(
    const void* __restrict__ q, int q_dt, const void* __restrict__ kc, const void* __restrict__ vc, int cache_dt,
    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_entry,
    const int* __restrict__ positions, float scale, int window, int has_sink, float sink_score,
    void* __restrict__ out, int out_dt, int Hq, int Hkv, int D, int Dv, int page) {
  __shared__ float qs[256];
  __shared__ float p[ATTG_THREADS];
  __shared__ int pslot[ATTG_THREADS];
  __shared__ float red[ATTG_THREADS / 32];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kvh = h / (Hq / Hkv);
  const int n = positions[t] + 1;
  const int lo = window > 0 ? max(0, n - window) : 0;
  const int* bt = block_table + (size_t)row_entry[t] * max_blocks;
  for (int d = tid; d < D; d += ATTG_THREADS) qs[d] = ld_dt(q, q_dt, (size_t)t * Hq * D + (size_t)h * D + d);
  __syncthreads();
  float m = has_sink ? sink_score : -1e30f, l = has_sink ? 1.f : 0.f;
  float o0 = 0.f, o1 = 0.f;          // output elements tid and tid + ATTG_THREADS
  for (int c0 = lo; c0 < n; c0 += ATTG_THREADS) {
    const int j = c0 + tid;
    float s = -1e30f;
    if (j < n) {
      const int blk = bt[j / page];
      const size_t slot = ((size_t)blk * Hkv + kvh) * page + j % page;
      pslot[tid] = (int)slot;
      float acc = 0.f;
      for (int d = 0; d < D; ++d) acc = fmaf(qs[d], ld_dt(kc, cache_dt, slot * D + d), acc);
      s = acc * scale;
    }
    // maximum over the chunk
    float mx = warp_max(s);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < ATTG_THREADS / 32; ++i) mx = fmaxf(mx, red[i]);
    const float m_new = fmaxf(m, mx);
    const float ex = j < n ? expf(s - m_new) : 0.f;
    p[tid] = ex;
    float sum = warp_sum(ex);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = sum;
    __syncthreads();
    sum = 0.f;
    for (int i = 0; i < ATTG_THREADS / 32; ++i) sum += red[i];
    const float alpha = expf(m - m_new);
    l = l * alpha + sum;
    m = m_new;
    const int cnt = min(ATTG_THREADS, n - c0);
    o0 *= alpha;
    o1 *= alpha;
    if (tid < Dv)
      for (int i = 0; i < cnt; ++i) o0 = fmaf(p[i], ld_dt(vc, cache_dt, (size_t)pslot[i] * Dv + tid), o0);
    if (tid + ATTG_THREADS < Dv)
      for (int i = 0; i < cnt; ++i) o1 = fmaf(p[i], ld_dt(vc, cache_dt, (size_t)pslot[i] * Dv + tid + ATTG_THREADS), o1);
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const size_t ob = (size_t)t * Hq * Dv + (size_t)h * Dv;
  if (tid < Dv) st_dt(out, out_dt, ob + tid, o0 * inv);
  if (tid + ATTG_THREADS < Dv) st_dt(out, out_dt, ob + tid + ATTG_THREADS, o1 * inv);
}

size_t scan_smem(int dk, int dv, int parts) {
  const int RS = std::max(1, std::min(SM_THREADS / dv, dk));
  return sizeof(float) * ((size_t)dk * dv + 3 * (size_t)dk + (size_t)(2 + parts) * dv + (size_t)parts * RS * dv + 8);
}

template <typename K>
int allow_smem(K kernel, size_t bytes) {
  if (bytes > 227 * 1024) return NV_ERR_UNSUPPORTED;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return NV_OK;
}

}  // namespace

NV_API int nv_branch_norm_add(float* x, const float* b0, const float* b1, const float* b2, const float* b3,
                              const float* w0, const float* w1, const float* w2, const float* w3, int nb,
                              float mix_scale, const float* w, float eps, void* out, int out_dt, int T, int H,
                              cudaStream_t s) {
  if (nb < 0 || nb > MAX_BRANCHES || H <= 0) return NV_ERR_BAD_SIZE;
  if (out && !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (T == 0) return NV_OK;
  BranchArgs a;
  a.x = x;
  const float* br[4] = {b0, b1, b2, b3};
  const float* bw[4] = {w0, w1, w2, w3};
  for (int i = 0; i < MAX_BRANCHES; ++i) { a.br[i] = br[i]; a.bw[i] = bw[i]; }
  for (int i = 0; i < nb; ++i) {
    if (!br[i]) return NV_ERR_BAD_SIZE;
    if ((bw[i] != nullptr) != (bw[0] != nullptr)) return NV_ERR_BAD_SIZE;
  }
  if (nb > 1 && !bw[0]) return NV_ERR_BAD_SIZE;
  if (nb > 0 && !w) return NV_ERR_BAD_SIZE;
  a.w = w; a.out = out; a.nb = nb; a.H = H; a.out_dt = out_dt; a.eps = eps; a.mix_scale = mix_scale;
  const size_t smem = sizeof(float) * (size_t)H;
  int rc = allow_smem(branch_norm_add_kernel, smem);
  if (rc) return rc;
  branch_norm_add_kernel<<<T, SM_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_activation(const void* in, int in_dt, void* out, int out_dt, long long n, int kind, cudaStream_t s) {
  if (!dt_ok(in_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (kind < 0 || kind > 2) return NV_ERR_UNSUPPORTED;
  if (n == 0) return NV_OK;
  activation_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(in, in_dt, out, out_dt, n, kind);
  NV_RETURN_LAST();
}

NV_API int nv_token_gate(const void* gate, int gate_dt, long long gate_ld, const int* ids, const int* feed,
                         const void* table, int table_dt, long long table_ld, int col0, int d, int V, void* out,
                         int out_dt, int T, int* err, cudaStream_t s) {
  if (!dt_ok(gate_dt) || !dt_ok(table_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (d <= 0 || col0 < 0 || col0 + d > table_ld) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  token_gate_kernel<<<T, 128, 0, s>>>(gate, gate_dt, gate_ld, ids, feed, table, table_dt, table_ld, col0, d, V, out,
                                      out_dt, err);
  NV_RETURN_LAST();
}

NV_API int nv_conv_silu_norm(const void* in, int in_dt, long long ld, int col0, int C, const float* w, int taps,
                             const int* row_entry, const int* cu_rows, const int* entry_slot, const float* state,
                             long long slot_stride, int unit_heads, int unit_dim, float unit_eps, int scaled_heads,
                             float scale, float* out, int T, cudaStream_t s) {
  if (!dt_ok(in_dt)) return NV_ERR_BAD_DTYPE;
  if (C <= 0 || taps < 1 || unit_heads < 0 || unit_heads * unit_dim > C || scaled_heads > unit_heads) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  const size_t smem = sizeof(float) * (size_t)C;
  int rc = allow_smem(conv_silu_norm_kernel, smem);
  if (rc) return rc;
  conv_silu_norm_kernel<<<T, SM_THREADS, smem, s>>>(in, in_dt, ld, col0, C, w, taps, row_entry, cu_rows, entry_slot,
                                                    state, slot_stride, unit_heads, unit_dim, unit_eps, scaled_heads,
                                                    scale, out);
  NV_RETURN_LAST();
}

NV_API int nv_conv_state_update(const void* in, int in_dt, long long ld, int col0, int C, int taps,
                                const int* cu_rows, const int* entry_slot, float* state, long long slot_stride,
                                int S, cudaStream_t s) {
  if (!dt_ok(in_dt)) return NV_ERR_BAD_DTYPE;
  if (C <= 0 || taps < 1) return NV_ERR_BAD_SIZE;
  if (S == 0 || taps == 1) return NV_OK;
  conv_state_update_kernel<<<S, SM_THREADS, 0, s>>>(in, in_dt, ld, col0, C, taps, cu_rows, entry_slot, state,
                                                    slot_stride);
  NV_RETURN_LAST();
}

NV_API int nv_scan_usable(int dk, int dv, int parts) {
  return dk >= 1 && dv >= 1 && dv <= SM_THREADS && scan_smem(dk, dv, parts) <= 227 * 1024;
}

NV_API int nv_mlstm_scan(const float* proj, long long ld, int q0, int k0, int v0, int g0, int i0, int f0,
                         const int* cu_rows, const int* entry_slot, float* S, long long S_stride, float* n,
                         long long n_stride, float* m, long long m_stride, int H, int dk, int dv, float cap,
                         float q_scale, float den_eps, float eps, const float* norm_w, int norm_per_head, void* out,
                         int out_dt, int num_entries, cudaStream_t s) {
  if (!dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (!nv_scan_usable(dk, dv, 1) || H <= 0) return NV_ERR_UNSUPPORTED;
  if (num_entries == 0) return NV_OK;
  MlstmArgs a;
  a.c = {cu_rows, entry_slot, S, S_stride, norm_w, out, out_dt, H, dk, dv, eps};
  a.proj = proj; a.ld = ld; a.q0 = q0; a.k0 = k0; a.v0 = v0; a.g0 = g0; a.i0 = i0; a.f0 = f0;
  a.n = n; a.n_stride = n_stride; a.m = m; a.m_stride = m_stride;
  a.cap = cap; a.q_scale = q_scale; a.den_eps = den_eps; a.norm_per_head = norm_per_head;
  const size_t smem = scan_smem(dk, dv, 1);
  int rc = allow_smem(mlstm_scan_kernel, smem);
  if (rc) return rc;
  mlstm_scan_kernel<<<dim3(num_entries, H), SM_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_gated_delta_scan(const float* qkv, int C, int q0, int k0, int v0, int G, const void* proj, int proj_dt,
                               long long ld, int g0, int b0, int a0, const float* A_log, const float* dt_bias,
                               const int* cu_rows, const int* entry_slot, float* S, long long S_stride, int H, int dk,
                               int dv, float eps, const float* norm_w, void* out, int out_dt, int num_entries,
                               cudaStream_t s) {
  if (!dt_ok(out_dt) || !dt_ok(proj_dt)) return NV_ERR_BAD_DTYPE;
  if (!nv_scan_usable(dk, dv, 2) || H <= 0 || G <= 0 || H % G) return NV_ERR_UNSUPPORTED;
  if (num_entries == 0) return NV_OK;
  DeltaArgs a;
  a.c = {cu_rows, entry_slot, S, S_stride, norm_w, out, out_dt, H, dk, dv, eps};
  a.qkv = qkv; a.C = C; a.q0 = q0; a.k0 = k0; a.v0 = v0; a.G = G;
  a.proj = proj; a.proj_dt = proj_dt; a.ld = ld; a.g0 = g0; a.b0 = b0; a.a0 = a0;
  a.A_log = A_log; a.dt_bias = dt_bias;
  const size_t smem = scan_smem(dk, dv, 2);
  int rc = allow_smem(gated_delta_scan_kernel, smem);
  if (rc) return rc;
  gated_delta_scan_kernel<<<dim3(num_entries, H), SM_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_qk_prepare_store(const void* in, int in_dt, long long ld, int q0, int k0, int v0, const int* positions,
                               const int* row_entry, const int* block_table, int max_blocks, const float* qw,
                               const float* kw, float eps, const float* inv_freq, int rot_dim, int interleaved,
                               float amplitude, void* q_out, int q_dt, void* kc, void* vc, int cache_dt, int Hq,
                               int Hkv, int D, int Dv, int page, int write_kv, int* err, int T, cudaStream_t s) {
  if (!dt_ok(in_dt) || !dt_ok(q_dt) || !dt_ok(cache_dt)) return NV_ERR_BAD_DTYPE;
  if (rot_dim < 0 || rot_dim > D || rot_dim % 2 || D <= 0 || Dv <= 0) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  QkArgs a = {in, in_dt, ld, q0, k0, v0, positions, row_entry, block_table, max_blocks, qw, kw, eps, inv_freq, rot_dim,
              interleaved, amplitude, q_out, q_dt, kc, vc, cache_dt, Hq, Hkv, D, Dv, page, write_kv, err};
  const size_t smem = sizeof(float) * (size_t)(QK_THREADS / 32) * D;
  int rc = allow_smem(qk_prepare_store_kernel, smem);
  if (rc) return rc;
  qk_prepare_store_kernel<<<T, QK_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_paged_attention_general(const void* q, int q_dt, const void* kc, const void* vc, int cache_dt,
                                      const int* block_table, int max_blocks, const int* row_entry,
                                      const int* positions, float scale, int window, int has_sink, float sink_score,
                                      void* out, int out_dt, int T, int Hq, int Hkv, int D, int Dv, int page,
                                      cudaStream_t s) {
  if (!dt_ok(q_dt) || !dt_ok(cache_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (D > 256 || D <= 0 || Dv <= 0 || Dv > 2 * ATTG_THREADS || Hkv <= 0 || Hq % Hkv) return NV_ERR_UNSUPPORTED;
  if (T == 0) return NV_OK;
  paged_attention_general_kernel<<<dim3(T, Hq), ATTG_THREADS, 0, s>>>(q, q_dt, kc, vc, cache_dt, block_table,
                                                                      max_blocks, row_entry, positions, scale, window,
                                                                      has_sink, sink_score, out, out_dt, Hq, Hkv, D,
                                                                      Dv, page);
  NV_RETURN_LAST();
}
