// Linear attention with a constant decay per head ("lightning attention"), and the gated norm behind it.
//
// Per head, with a state S [dk, dv] in 32 bit that a request carries from token to token:
//     S_t = lambda * S_(t-1) + k_t v_t^T ,      o_t = S_t^T q_t .
// A row's new tokens are taken in chunks of C.  With the chunk's tokens numbered 0..n-1 and S the state before it,
//     o_t = lambda^(t+1) * S^T q_t + sum_{s<=t} lambda^(t-s) (q_t . k_s) v_s
//     S  <- lambda^n * S + sum_s lambda^(n-1-s) k_s v_s^T
// which is the recurrence itself, summed in another order.  No power of lambda is ever divided by: the powers
// lambda^0..lambda^C are tabulated from the 64-bit decay.  q, k and v may get an activation (silu) as they are read;
// all arithmetic is 32-bit FMA, whatever the type of the inputs.
//
// decay_attention: one block per (row, head, slice of the value entries); the slice's part of the state stays in
// shared memory over the row's chunks and goes back to the request's slot at the end.
// gated_rms_norm:  out = rmsnorm(o over all heads) * w * sigmoid(gate), one block per token.
#include "common.cuh"

namespace {
constexpr int C = 32;            // tokens of a chunk
constexpr int THREADS = 256;

__device__ __forceinline__ float act_silu(float z) { return z / (1.f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(THREADS)
decay_attention_kernel(const T* __restrict__ src, int src_stride, int q_off, int k_off, int v_off, int act,
                       const double* __restrict__ decays, float* __restrict__ state, float* __restrict__ out,
                       const int* __restrict__ row_slot, const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                       int H, int dk, int dv, int dvs) {
  extern __shared__ __align__(16) float sm[];
  const int kp = dk + 1;                    // padded row of Q and K
  float* S = sm;                            // [dk][dvs]
  float* Q = S + (size_t)dk * dvs;          // [C][kp]
  float* K = Q + C * kp;                    // [C][kp]
  float* V = K + C * kp;                    // [C][dvs]
  float* A = V + C * dvs;                   // [C][C + 1]
  float* pw = A + C * (C + 1);              // [C + 1]
  const int row = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * dvs;
  const int jn = min(dvs, dv - j0);
  const int tid = threadIdx.x;
  const int n_new = row_q_len[row];
  if (n_new <= 0 || jn <= 0) return;
  const int t0 = row_q_start[row];
  float* st = state + (((size_t)row_slot[row] * H + h) * dk) * dv + j0;
  if (tid <= C) pw[tid] = (float)pow(decays[h], (double)tid);
  for (int idx = tid; idx < dk * jn; idx += THREADS) {
    const int i = idx / jn, j = idx - i * jn;
    S[i * dvs + j] = st[(size_t)i * dv + j];
  }
  for (int c0 = 0; c0 < n_new; c0 += C) {
    const int n = min(C, n_new - c0);
    __syncthreads();
    for (int idx = tid; idx < n * dk; idx += THREADS) {
      const int t = idx / dk, i = idx - t * dk;
      const T* p = src + (size_t)(t0 + c0 + t) * src_stride + (size_t)h * dk + i;
      const float qv = to_f32<T>(p[q_off]), kv = to_f32<T>(p[k_off]);
      Q[t * kp + i] = act ? act_silu(qv) : qv;
      K[t * kp + i] = act ? act_silu(kv) : kv;
    }
    for (int idx = tid; idx < n * jn; idx += THREADS) {
      const int t = idx / jn, j = idx - t * jn;
      const float vv = to_f32<T>(src[(size_t)(t0 + c0 + t) * src_stride + v_off + (size_t)h * dv + j0 + j]);
      V[t * dvs + j] = act ? act_silu(vv) : vv;
    }
    __syncthreads();
    // A[t][s] = lambda^(t-s) q_t . k_s for s <= t
    for (int idx = tid; idx < n * n; idx += THREADS) {
      const int t = idx / n, s = idx - t * n;
      if (s > t) continue;
      const float* qt = Q + t * kp;
      const float* ks = K + s * kp;
      float a = 0.f;
      for (int i = 0; i < dk; ++i) a = fmaf(qt[i], ks[i], a);
      A[t * (C + 1) + s] = a * pw[t - s];
    }
    __syncthreads();
    // o_t[j] = lambda^(t+1) sum_i q_t[i] S[i][j] + sum_{s<=t} A[t][s] v_s[j]
    for (int idx = tid; idx < n * jn; idx += THREADS) {
      const int t = idx / jn, j = idx - t * jn;
      const float* qt = Q + t * kp;
      float far = 0.f;
      for (int i = 0; i < dk; ++i) far = fmaf(qt[i], S[i * dvs + j], far);
      float near = 0.f;
      for (int s = 0; s <= t; ++s) near = fmaf(A[t * (C + 1) + s], V[s * dvs + j], near);
      out[(size_t)(t0 + c0 + t) * ((size_t)H * dv) + (size_t)h * dv + j0 + j] = fmaf(pw[t + 1], far, near);
    }
    __syncthreads();
    // S[i][j] = lambda^n S[i][j] + sum_s lambda^(n-1-s) k_s[i] v_s[j]
    for (int idx = tid; idx < dk * jn; idx += THREADS) {
      const int i = idx / jn, j = idx - i * jn;
      float a = 0.f;
      for (int s = 0; s < n; ++s) a = fmaf(pw[n - 1 - s] * K[s * kp + i], V[s * dvs + j], a);
      S[i * dvs + j] = fmaf(pw[n], S[i * dvs + j], a);
    }
  }
  __syncthreads();
  for (int idx = tid; idx < dk * jn; idx += THREADS) {
    const int i = idx / jn, j = idx - i * jn;
    st[(size_t)i * dv + j] = S[i * dvs + j];
  }
}

template <typename T>
__global__ void gated_rms_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                                      const float* __restrict__ w, T* __restrict__ out, int n, float eps) {
  __shared__ float scratch[34];
  const int t = blockIdx.x;
  const float* x = o + (size_t)t * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += x[i] * x[i];
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float g = to_f32<T>(gate[(size_t)t * gate_stride + i]);
    out[(size_t)t * n + i] = from_f32<T>(x[i] * inv * w[i] * (1.f / (1.f + expf(-g))));
  }
}

size_t smem_floats(int dk, int dvs) { return (size_t)dk * dvs + 2 * (size_t)C * (dk + 1) + (size_t)C * dvs + C * (C + 1) + C + 1; }
constexpr size_t SMEM_LIMIT = 200 * 1024;
}  // namespace

// The slice of value entries a block takes: the whole head when its state fits the shared memory, and a smaller one
// while the grid would leave SMs without a block.
extern "C" int dk_decay_attention_slice(int rows, int H, int dk, int dv) {
  int dvs = dv;
  while (dvs > 1 && smem_floats(dk, dvs) * sizeof(float) > SMEM_LIMIT) dvs = (dvs + 1) / 2;
  const int sms = dk_sm_count();
  while (dvs > 32 && (long long)rows * H * ((dv + dvs - 1) / dvs) < sms) dvs = (dvs + 1) / 2;
  return dvs;
}

extern "C" int dk_decay_attention(const void* src, int src_stride, int q_off, int k_off, int v_off, int act, const double* decays,
                                  float* state, float* out, const int* row_slot, const int* row_q_start, const int* row_q_len,
                                  int rows, int H, int dk, int dv, int dvs, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && H > 0 && dk > 0 && dv > 0 && dvs > 0 && dvs <= dv, "decay_attention: bad sizes rows=%d H=%d dk=%d dv=%d slice=%d", rows, H, dk, dv, dvs);
  const size_t smem = smem_floats(dk, dvs) * sizeof(float);
  DK_REQUIRE(smem <= SMEM_LIMIT, "decay_attention: a state slice of %d x %d does not fit the shared memory", dk, dvs);
  DK_REQUIRE(H <= 65535, "decay_attention: %d heads are above the grid's limit", H);
  const dim3 grid(rows, H, (dv + dvs - 1) / dvs);
#define LAUNCH(T)                                                                                                                   \
  do {                                                                                                                              \
    if (smem > 48 * 1024 &&                                                                                                         \
        cudaFuncSetAttribute(decay_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { \
      cudaGetLastError();                                                                                                           \
      DK_REQUIRE(false, "decay_attention: %zu bytes of shared memory were not granted", smem);                                      \
    }                                                                                                                               \
    decay_attention_kernel<T><<<grid, THREADS, smem, stream>>>((const T*)src, src_stride, q_off, k_off, v_off, act, decays, state,  \
                                                                out, row_slot, row_q_start, row_q_len, H, dk, dv, dvs);            \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "decay_attention: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("decay_attention");
}

extern "C" int dk_gated_rms_norm(const float* o, const void* gate, int gate_stride, const float* w, void* out, int T_, int n, float eps,
                                 int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && n > 0 && gate_stride >= n, "gated_rms_norm: bad sizes T=%d n=%d stride=%d", T_, n, gate_stride);
  const int threads = n >= 2048 ? 256 : 128;
  if (dtype == DK_F32)
    gated_rms_norm_kernel<float><<<T_, threads, 0, stream>>>(o, (const float*)gate, gate_stride, w, (float*)out, n, eps);
  else if (dtype == DK_BF16)
    gated_rms_norm_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(o, (const __nv_bfloat16*)gate, gate_stride, w, (__nv_bfloat16*)out, n, eps);
  else DK_REQUIRE(false, "gated_rms_norm: unknown dtype %d", dtype);
  return dk_check_launch("gated_rms_norm");
}
