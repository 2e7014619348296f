// A mixture of small feed-forward experts, and the gated activation its experts and dense layers share.
//
//   glu_clamped     y = g' * sigmoid(alpha g') * (u' + shift),  g' = min(g, limit), u' = clamp(u, -limit, limit)
//                   from rows [g (F) | u (F)] (limit < 0: nothing is clamped);
//   router_topk     per token the `top` largest of E router logits (32 bit; the lowest index among equals) and the
//                   softmax over the chosen logits only;
//   experts_align   sorts the (token, choice) slots by expert into tiles of TILE_M rows that each belong to one expert
//                   (every expert's rows padded to whole tiles with -1), so that the products run as one launch and
//                   nothing about the routing is read on the host;
//   experts_gemm    for every tile the product of its rows with its expert's matrix.  First product: rows are gathered
//                   from the tokens, the matrix is [gate (F) | up (F)] x d, and the gated activation is applied before
//                   the result is stored at the row's place in the sorted order.  Second product: rows are read in the
//                   sorted order and the result goes to the slot's own place, in 32 bit;
//   experts_combine out[t] = sum_j weight[t][j] * z[t*top + j]  (+ sigmoid(gate logit of t) * shared[t]), summed in 32 bit in
//                   the order of the choices, so the result does not depend on what else is in the batch.
//
// The products here run on the FMA units with 32-bit accumulation for both element types.
#include "common.cuh"

namespace {
constexpr int TILE_M = 32;
constexpr int TILE_N = 64;
constexpr int TILE_K = 16;
constexpr int GEMM_THREADS = 256;
constexpr int MAX_TOP = 32;
constexpr int MAX_EXPERTS = 1024;

__device__ __forceinline__ float glu_value(float g, float u, float limit, float alpha, float shift) {
  if (limit >= 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return g * (1.f / (1.f + expf(-alpha * g))) * (u + shift);
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ y, long long rows, int F, float limit, float alpha, float shift) {
  const long long n = rows * F;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / F;
    const int i = (int)(idx - r * F);
    const T* row = gu + r * 2 * F;
    y[idx] = from_f32<T>(glu_value(to_f32<T>(row[i]), to_f32<T>(row[F + i]), limit, alpha, shift));
  }
}

__global__ void router_topk_kernel(const float* __restrict__ logits, int ld, int* __restrict__ choice, float* __restrict__ weight, int T_,
                                   int E, int top) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T_) return;
  const float* z = logits + (size_t)t * ld;
  int picked[MAX_TOP];
  float val[MAX_TOP];
  for (int j = 0; j < top; ++j) {
    int best = -1;
    float bv = 0.f;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int q = 0; q < j; ++q) taken |= picked[q] == e;
      if (taken) continue;
      const float v = z[e];
      if (best < 0 || v > bv) {
        best = e;
        bv = v;
      }
    }
    picked[j] = best;
    val[j] = bv;
  }
  float sum = 0.f;
  const float largest = val[0];
  for (int j = 0; j < top; ++j) {
    val[j] = expf(val[j] - largest);
    sum += val[j];
  }
  for (int j = 0; j < top; ++j) {
    choice[(size_t)t * top + j] = picked[j];
    weight[(size_t)t * top + j] = val[j] / sum;
  }
}

// One block.  sorted[p] = slot (token * top + choice) or -1; tile_expert[tile] = expert or -1.
__global__ void experts_align_kernel(const int* __restrict__ choice, int n_slots, int E, int* __restrict__ sorted, int capacity,
                                     int* __restrict__ tile_expert, int max_tiles) {
  __shared__ int count[MAX_EXPERTS], start[MAX_EXPERTS];
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
    const int e = choice[s];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  for (int p = threadIdx.x; p < capacity; p += blockDim.x) sorted[p] = -1;
  for (int q = threadIdx.x; q < max_tiles; q += blockDim.x) tile_expert[q] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      const int tiles = (count[e] + TILE_M - 1) / TILE_M;
      for (int q = 0; q < tiles; ++q) tile_expert[at / TILE_M + q] = e;
      at += tiles * TILE_M;
      count[e] = 0;
    }
  }
  __syncthreads();
  // the order of an expert's rows is whatever the atomics give: every row is computed alone, so it changes no value
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
    const int e = choice[s];
    if (e < 0 || e >= E) continue;
    sorted[start[e] + atomicAdd(&count[e], 1)] = s;
  }
}

// ACT: A = tokens [*, K] gathered by sorted[p] / top, W = [E][2N][K] (gate rows, then up rows), out Y[p][N] of type T.
// !ACT: A = Y [capacity, K] in sorted order, W = [E][N][K], out Z[slot][N] in float.
template <typename T, bool ACT>
__global__ void __launch_bounds__(GEMM_THREADS)
experts_gemm_kernel(const T* __restrict__ A, const T* __restrict__ W, void* __restrict__ out, const int* __restrict__ sorted,
                    const int* __restrict__ tile_expert, int top, int N, int K, float limit, float alpha, float shift) {
  const int tile = blockIdx.y;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int n0 = blockIdx.x * TILE_N, p0 = tile * TILE_M;
  __shared__ float As[TILE_M][TILE_K + 1];
  __shared__ float Ws[ACT ? 2 : 1][TILE_N][TILE_K + 1];
  __shared__ int src_row[TILE_M];
  const int tid = threadIdx.x;
  if (tid < TILE_M) {
    const int s = sorted[p0 + tid];
    src_row[tid] = s < 0 ? -1 : (ACT ? s / top : p0 + tid);
  }
  __syncthreads();
  const T* We = W + (size_t)e * (ACT ? 2 : 1) * N * K;
  const int ty = tid / 16, tx = tid % 16;      // rows 2*ty, 2*ty+1; columns tx + 16*c
  float acc[ACT ? 2 : 1][2][4];
#pragma unroll
  for (int a = 0; a < (ACT ? 2 : 1); ++a)
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][r][c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TILE_K) {
    for (int idx = tid; idx < TILE_M * TILE_K; idx += GEMM_THREADS) {
      const int r = idx / TILE_K, k = idx - r * TILE_K;
      const int row = src_row[r];
      As[r][k] = (row >= 0 && k0 + k < K) ? to_f32<T>(A[(size_t)row * K + k0 + k]) : 0.f;
    }
    for (int idx = tid; idx < TILE_N * TILE_K; idx += GEMM_THREADS) {
      const int c = idx / TILE_K, k = idx - c * TILE_K;
      const bool ok = n0 + c < N && k0 + k < K;
      Ws[0][c][k] = ok ? to_f32<T>(We[(size_t)(n0 + c) * K + k0 + k]) : 0.f;
      if (ACT) Ws[ACT ? 1 : 0][c][k] = ok ? to_f32<T>(We[(size_t)(N + n0 + c) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TILE_K; ++k) {
      const float a0 = As[2 * ty][k], a1 = As[2 * ty + 1][k];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float w0 = Ws[0][tx + 16 * c][k];
        acc[0][0][c] = fmaf(a0, w0, acc[0][0][c]);
        acc[0][1][c] = fmaf(a1, w0, acc[0][1][c]);
        if (ACT) {
          const float w1 = Ws[ACT ? 1 : 0][tx + 16 * c][k];
          acc[ACT ? 1 : 0][0][c] = fmaf(a0, w1, acc[ACT ? 1 : 0][0][c]);
          acc[ACT ? 1 : 0][1][c] = fmaf(a1, w1, acc[ACT ? 1 : 0][1][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int lr = 2 * ty + r;
    const int s = sorted[p0 + lr];
    if (s < 0) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx + 16 * c;
      if (n >= N) continue;
      if (ACT) {
        // the two products are rounded to the element type before the activation, as separate products would be
        const float g = to_f32<T>(from_f32<T>(acc[0][r][c])), u = to_f32<T>(from_f32<T>(acc[ACT ? 1 : 0][r][c]));
        ((T*)out)[(size_t)(p0 + lr) * N + n] = from_f32<T>(glu_value(g, u, limit, alpha, shift));
      } else {
        ((float*)out)[(size_t)s * N + n] = acc[0][r][c];
      }
    }
  }
}

template <typename T>
__global__ void experts_combine_kernel(const float* __restrict__ z, const float* __restrict__ weight, int top, const T* __restrict__ shared,
                                       const float* __restrict__ gate_logit, int gate_stride, T* __restrict__ out, int d) {
  const int t = blockIdx.x;
  float gate = 0.f;
  if (shared != nullptr) gate = gate_logit != nullptr ? 1.f / (1.f + expf(-gate_logit[(size_t)t * gate_stride])) : 1.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < top; ++j) a = fmaf(weight[(size_t)t * top + j], z[((size_t)t * top + j) * d + i], a);
    if (shared != nullptr) a = fmaf(gate, to_f32<T>(shared[(size_t)t * d + i]), a);
    out[(size_t)t * d + i] = from_f32<T>(a);
  }
}
}  // namespace

extern "C" int dk_experts_tile_rows() { return TILE_M; }

extern "C" int dk_glu_clamped(const void* gu, void* y, long long rows, int F, float limit, float alpha, float shift, int dtype,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && F > 0, "glu_clamped: bad sizes rows=%lld F=%d", rows, F);
  const long long n = rows * F;
  long long blocks = (n + 255) / 256;
  const long long most = (long long)dk_sm_count() * 16;
  if (blocks > most) blocks = most;
  if (dtype == DK_F32) glu_clamped_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)gu, (float*)y, rows, F, limit, alpha, shift);
  else if (dtype == DK_BF16)
    glu_clamped_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)y, rows, F, limit, alpha, shift);
  else DK_REQUIRE(false, "glu_clamped: unknown dtype %d", dtype);
  return dk_check_launch("glu_clamped");
}

extern "C" int dk_router_topk(const float* logits, int ld, int* choice, float* weight, int T_, int E, int top, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && E > 0 && top > 0 && top <= E && ld >= E, "router_topk: bad sizes T=%d E=%d top=%d ld=%d", T_, E, top, ld);
  DK_REQUIRE(top <= MAX_TOP, "router_topk: %d choices a token are above the %d this kernel takes", top, MAX_TOP);
  router_topk_kernel<<<(T_ + 63) / 64, 64, 0, stream>>>(logits, ld, choice, weight, T_, E, top);
  return dk_check_launch("router_topk");
}

extern "C" int dk_experts_align(const int* choice, int n_slots, int E, int* sorted, int capacity, int* tile_expert, int max_tiles,
                                cudaStream_t stream) {
  if (n_slots == 0) return 0;
  DK_REQUIRE(n_slots > 0 && E > 0 && E <= MAX_EXPERTS, "experts_align: bad sizes slots=%d E=%d (at most %d experts)", n_slots, E, MAX_EXPERTS);
  DK_REQUIRE(capacity % TILE_M == 0 && max_tiles * TILE_M == capacity && capacity >= n_slots + (TILE_M - 1) * (E < n_slots ? E : n_slots),
             "experts_align: %d rows in %d tiles do not hold %d slots of %d experts", capacity, max_tiles, n_slots, E);
  experts_align_kernel<<<1, 1024, 0, stream>>>(choice, n_slots, E, sorted, capacity, tile_expert, max_tiles);
  return dk_check_launch("experts_align");
}

extern "C" int dk_experts_gemm(const void* A, const void* W, void* out, const int* sorted, const int* tile_expert, int max_tiles, int top,
                               int N, int K, int act, float limit, float alpha, float shift, int dtype, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  DK_REQUIRE(max_tiles > 0 && N > 0 && K > 0 && top > 0, "experts_gemm: bad sizes tiles=%d N=%d K=%d top=%d", max_tiles, N, K, top);
  DK_REQUIRE(max_tiles <= 65535, "experts_gemm: %d tiles are above the grid's limit", max_tiles);
  const dim3 grid((N + TILE_N - 1) / TILE_N, max_tiles);
#define LAUNCH(T)                                                                                                                  \
  do {                                                                                                                             \
    if (act) experts_gemm_kernel<T, true><<<grid, GEMM_THREADS, 0, stream>>>((const T*)A, (const T*)W, out, sorted, tile_expert, top, N, K, limit, alpha, shift); \
    else experts_gemm_kernel<T, false><<<grid, GEMM_THREADS, 0, stream>>>((const T*)A, (const T*)W, out, sorted, tile_expert, top, N, K, limit, alpha, shift);    \
  } while (0)
  if (dtype == DK_F32) LAUNCH(float);
  else if (dtype == DK_BF16) LAUNCH(__nv_bfloat16);
  else DK_REQUIRE(false, "experts_gemm: unknown dtype %d", dtype);
#undef LAUNCH
  return dk_check_launch("experts_gemm");
}

extern "C" int dk_experts_combine(const float* z, const float* weight, int top, const void* shared, const float* gate_logit,
                                  int gate_stride, void* out, int T_, int d, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  DK_REQUIRE(T_ > 0 && d > 0 && top > 0, "experts_combine: bad sizes T=%d d=%d top=%d", T_, d, top);
  const int threads = d >= 1024 ? 256 : 128;
  if (dtype == DK_F32)
    experts_combine_kernel<float><<<T_, threads, 0, stream>>>(z, weight, top, (const float*)shared, gate_logit, gate_stride, (float*)out, d);
  else if (dtype == DK_BF16)
    experts_combine_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(z, weight, top, (const __nv_bfloat16*)shared, gate_logit, gate_stride,
                                                                      (__nv_bfloat16*)out, d);
  else DK_REQUIRE(false, "experts_combine: unknown dtype %d", dtype);
  return dk_check_launch("experts_combine");
}
