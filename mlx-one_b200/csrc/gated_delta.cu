// The gated delta rule over a ragged batch, with per-request state in 32-bit slots.
//
// projected[t] = [q: G x D | k: G x D | v: H x V | gate: H x V | beta: H | decay: H] (G query/key
// heads of D values, H value heads of V values; value head h reads query/key head h / (H / G)).
// The first C = 2 G D + H V channels pass a causal convolution over the last `taps` tokens of the
// request (conv [C, taps], last column the current token's) and silu.
//
// A request's slot holds, in 32-bit: S [H, D, V], then the convolution's last taps - 1 inputs
// [taps - 1, C] (row s is the input at position history - (taps - 1) + s).
//
// Three kernels:
//   prepare  per token: convolution + silu; q and k to unit length per head (q also times
//            D^-1/2); beta = sigmoid, g = exp(-exp(A_log) softplus(a + dt_bias)); k.q per head.
//   scan     per (request, value head, tile of columns of S): for each token of the request, in
//            order:  S = g S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q.
//            A column of S depends on no other column, so columns are spread over threads and
//            blocks; a column's D values are spread over four lanes of a warp. With the dot
//            products of the column with k and q taken before the update,
//            u = beta (v - g (S.k)) and o = g (S.q) + u (k.q): one pass reads the column for both
//            sums and a second one updates it. Extra blocks move the convolution's inputs
//            into the slot.
//   finish   per (token, head): o / rms(o) * weight * silu(gate), in the compute type.
#include "common.cuh"

namespace {

constexpr int PREP_THREADS = 256;
constexpr int LANES = 4;             // lanes that share a column of S
constexpr int COLUMNS = 32;          // columns of S per block
constexpr int SCAN_THREADS = LANES * COLUMNS;
constexpr int CHUNK = 16;            // tokens whose operands are staged in shared memory together

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct DeltaSizes {
    int heads, kv_heads, key_dim, value_dim, taps;
    __host__ __device__ int qk() const { return kv_heads * key_dim; }
    __host__ __device__ int inner() const { return heads * value_dim; }
    __host__ __device__ int channels() const { return 2 * qk() + inner(); }
    __host__ __device__ int width() const { return channels() + inner() + 2 * heads; }
    __host__ __device__ long long matrices() const { return (long long)heads * key_dim * value_dim; }
    __host__ __device__ long long state() const {
        return matrices() + (long long)(taps - 1) * channels();
    }
};

// ------------------------------------------------------------------ prepare
// One block per token. q_out, k_out [tokens, G, D]; v_out [tokens, H, V]; coef [tokens, H, 2] =
// (g, beta); kq [tokens, G].
template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
delta_prepare_kernel(const T* __restrict__ projected, const float* __restrict__ conv,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const float* __restrict__ state, const int* __restrict__ slots,
                     const int* __restrict__ token_request, const int* __restrict__ request_start,
                     const int* __restrict__ history, float* __restrict__ q_out,
                     float* __restrict__ k_out, float* __restrict__ v_out, float* __restrict__ coef,
                     float* __restrict__ kq, DeltaSizes sizes, float unit_eps) {
    extern __shared__ float mixed[];                 // the token's C channels after conv + silu
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int r = token_request[t];
    const int index = t - request_start[r];
    const int position = history[r] + index;
    const int taps = sizes.taps, channels = sizes.channels(), width = sizes.width();
    const float* tail = state + (size_t)slots[r] * sizes.state() + sizes.matrices();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;
            float x = 0.f;
            if (index - back >= 0)
                x = to_float<T>(projected[(size_t)(t - back) * width + c]);
            else if (position - back >= 0)
                x = tail[(size_t)(taps - 1 + index - back) * channels + c];
            y = fmaf(conv[(size_t)c * taps + j], x, y);
        }
        mixed[c] = silu(y);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int G = sizes.kv_heads, D = sizes.key_dim, H = sizes.heads, V = sizes.value_dim;
    // queries and keys: a warp per head
    for (int g = warp; g < G; g += warps) {
        const float* q = mixed + (size_t)g * D;
        const float* k = mixed + (size_t)sizes.qk() + (size_t)g * D;
        float qq = 0.f, kk = 0.f;
        for (int e = lane; e < D; e += 32) {
            qq = fmaf(q[e], q[e], qq);
            kk = fmaf(k[e], k[e], kk);
        }
        qq = warp_sum(qq);
        kk = warp_sum(kk);
        const float q_scale = rsqrtf((float)D) / sqrtf(qq + unit_eps);
        const float k_scale = 1.f / sqrtf(kk + unit_eps);
        float dot = 0.f;
        for (int e = lane; e < D; e += 32) {
            const float qv = q[e] * q_scale, kv = k[e] * k_scale;
            q_out[((size_t)t * G + g) * D + e] = qv;
            k_out[((size_t)t * G + g) * D + e] = kv;
            dot = fmaf(qv, kv, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) kq[(size_t)t * G + g] = dot;
    }
    for (int c = threadIdx.x; c < H * V; c += blockDim.x)
        v_out[(size_t)t * H * V + c] = mixed[2 * sizes.qk() + c];
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        const T* row = projected + (size_t)t * width + channels + sizes.inner();
        const float beta = 1.f / (1.f + expf(-to_float<T>(row[h])));
        const float step = softplus(to_float<T>(row[H + h]) + dt_bias[h]);
        coef[((size_t)t * H + h) * 2] = expf(-expf(a_log[h]) * step);
        coef[((size_t)t * H + h) * 2 + 1] = beta;
    }
}

// ------------------------------------------------------------------ scan
// Grid (column tiles, H + 1, requests); blocks with blockIdx.y == H move the convolution's
// inputs. A thread keeps PER values of its column: element e of lane l is row
// (e / 4) * 16 + l * 4 + e % 4 of S, so that the four lanes read k and q as neighbouring float4.
template <typename T, int PER>
__global__ void __launch_bounds__(SCAN_THREADS)
delta_scan_kernel(const float* __restrict__ q_in, const float* __restrict__ k_in,
                  const float* __restrict__ v_in, const float* __restrict__ coef,
                  const float* __restrict__ kq, const T* __restrict__ projected,
                  float* __restrict__ state, const int* __restrict__ slots,
                  const int* __restrict__ request_start, float* __restrict__ out, DeltaSizes sizes,
                  int write) {
    constexpr int ROWS = PER * LANES;                 // rows of S a thread group covers (>= D)
    __shared__ __align__(16) float ks[CHUNK][ROWS];
    __shared__ __align__(16) float qs[CHUNK][ROWS];
    __shared__ float vs[CHUNK][COLUMNS];
    __shared__ float gs[CHUNK], bs[CHUNK], kqs[CHUNK];
    griddep_launch();
    griddep_wait();
    const int r = blockIdx.z;
    const int first = request_start[r], last = request_start[r + 1];
    const int H = sizes.heads, G = sizes.kv_heads, D = sizes.key_dim, V = sizes.value_dim;
    float* slot = state + (size_t)slots[r] * sizes.state();
    if (blockIdx.y == H) {
        // the convolution's last taps - 1 inputs: rows of this step, or what the slot held
        if (!write || sizes.taps < 2) return;
        const int channels = sizes.channels(), width = sizes.width(), keep = sizes.taps - 1;
        const int n = last - first;
        float* tail = slot + sizes.matrices();
        for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels;
             c += gridDim.x * blockDim.x) {
            for (int s = 0; s < keep; ++s) {
                const int index = n - keep + s;       // place in the portion, may be negative
                float x;
                if (index >= 0) x = to_float<T>(projected[(size_t)(first + index) * width + c]);
                else x = tail[(size_t)(s + n) * channels + c];
                tail[(size_t)s * channels + c] = x;
            }
        }
        return;
    }
    const int h = blockIdx.y, g = h / (H / G);
    const int lane = threadIdx.x & (LANES - 1);
    const int column = blockIdx.x * COLUMNS + (threadIdx.x >> 2);
    const bool live = column < V;
    float* matrix = slot + (size_t)h * D * V;
    float S[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int row = (e / 4) * 16 + lane * 4 + e % 4;
        S[e] = live && row < D ? matrix[(size_t)row * V + column] : 0.f;
    }
    for (int base = first; base < last; base += CHUNK) {
        const int count = min(CHUNK, last - base);
        __syncthreads();
        for (int i = threadIdx.x; i < count * ROWS; i += SCAN_THREADS) {
            const int t = i / ROWS, e = i % ROWS;
            const size_t at = ((size_t)(base + t) * G + g) * D + e;
            ks[t][e] = e < D ? k_in[at] : 0.f;
            qs[t][e] = e < D ? q_in[at] : 0.f;
        }
        for (int i = threadIdx.x; i < count * COLUMNS; i += SCAN_THREADS) {
            const int t = i / COLUMNS, c = blockIdx.x * COLUMNS + i % COLUMNS;
            vs[t][i % COLUMNS] = c < V ? v_in[((size_t)(base + t) * H + h) * V + c] : 0.f;
        }
        if (threadIdx.x < count) {
            const size_t at = (size_t)(base + threadIdx.x) * H + h;
            gs[threadIdx.x] = coef[at * 2];
            bs[threadIdx.x] = coef[at * 2 + 1];
            kqs[threadIdx.x] = kq[(size_t)(base + threadIdx.x) * G + g];
        }
        __syncthreads();
        for (int t = 0; t < count; ++t) {
            float k[PER];
            float with_k = 0.f, with_q = 0.f;
#pragma unroll
            for (int e = 0; e < PER; e += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][(e / 4) * 16 + lane * 4]);
                const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][(e / 4) * 16 + lane * 4]);
                k[e] = k4.x; k[e + 1] = k4.y; k[e + 2] = k4.z; k[e + 3] = k4.w;
                with_k = fmaf(S[e], k4.x, with_k); with_q = fmaf(S[e], q4.x, with_q);
                with_k = fmaf(S[e + 1], k4.y, with_k); with_q = fmaf(S[e + 1], q4.y, with_q);
                with_k = fmaf(S[e + 2], k4.z, with_k); with_q = fmaf(S[e + 2], q4.z, with_q);
                with_k = fmaf(S[e + 3], k4.w, with_k); with_q = fmaf(S[e + 3], q4.w, with_q);
            }
            with_k += __shfl_xor_sync(0xffffffffu, with_k, 1);
            with_q += __shfl_xor_sync(0xffffffffu, with_q, 1);
            with_k += __shfl_xor_sync(0xffffffffu, with_k, 2);
            with_q += __shfl_xor_sync(0xffffffffu, with_q, 2);
            const float decay = gs[t];
            const float u = bs[t] * (vs[t][threadIdx.x >> 2] - decay * with_k);
#pragma unroll
            for (int e = 0; e < PER; ++e) S[e] = fmaf(k[e], u, decay * S[e]);
            if (live && lane == 0)
                out[((size_t)(base + t) * H + h) * V + column] = fmaf(u, kqs[t], decay * with_q);
        }
    }
    if (write && live) {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int row = (e / 4) * 16 + lane * 4 + e % 4;
            if (row < D) matrix[(size_t)row * V + column] = S[e];
        }
    }
}

// ------------------------------------------------------------------ finish
// One warp per (token, head): mixed[t, h, :] = o / sqrt(mean(o^2) + eps) * weight * silu(gate).
template <typename T>
__global__ void __launch_bounds__(256)
delta_finish_kernel(const float* __restrict__ o, const T* __restrict__ projected,
                    const float* __restrict__ weight, T* __restrict__ mixed, long long items,
                    DeltaSizes sizes, float eps) {
    griddep_launch();
    griddep_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const int H = sizes.heads, V = sizes.value_dim;
    const long long t = item / H;
    const int h = (int)(item % H);
    const float* row = o + item * V;
    const T* gate = projected + (size_t)t * sizes.width() + sizes.channels() + (size_t)h * V;
    float sum = 0.f;
    for (int e = lane; e < V; e += 32) sum = fmaf(row[e], row[e], sum);
    sum = warp_sum(sum);
    const float inv = 1.f / sqrtf(sum / (float)V + eps);
    for (int e = lane; e < V; e += 32)
        mixed[item * V + e] = from_float<T>(row[e] * inv * weight[e] * silu(to_float<T>(gate[e])));
}

template <typename T>
int launch_delta(const void* projected, const float* conv, const float* a_log, const float* dt_bias,
                 const float* norm_weight, float eps, float unit_eps, float* state,
                 const int* slots, const int* token_request, const int* request_start,
                 const int* history, float* scratch, void* mixed, int tokens, int requests,
                 DeltaSizes sizes, int write, cudaStream_t stream) {
    const int G = sizes.kv_heads, D = sizes.key_dim, H = sizes.heads, V = sizes.value_dim;
    // scratch: q, k [tokens, G, D]; v, o [tokens, H, V]; coef [tokens, H, 2]; kq [tokens, G]
    float* q = scratch;
    float* k = q + (size_t)tokens * G * D;
    float* v = k + (size_t)tokens * G * D;
    float* o = v + (size_t)tokens * H * V;
    float* coef = o + (size_t)tokens * H * V;
    float* kq = coef + (size_t)tokens * H * 2;
    const size_t shared = (size_t)sizes.channels() * sizeof(float);
    if (shared > 48 * 1024) {
        MLXONE_REQUIRE(shared <= 200 * 1024, "gated delta rule: %d channels do not fit",
                       sizes.channels());
        cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)shared);
    }
    launch_kernel(delta_prepare_kernel<T>, dim3(tokens), dim3(PREP_THREADS), shared, stream, true,
                  (const T*)projected, conv, a_log, dt_bias, (const float*)state, slots,
                  token_request, request_start, history, q, k, v, coef, kq, sizes, unit_eps);
    MLXONE_LAUNCH_CHECK("gated delta rule (prepare)");
    const dim3 grid(ceil_div_host(V, COLUMNS), H + 1, requests);
#define SCAN(PER)                                                                               \
    launch_kernel(delta_scan_kernel<T, PER>, grid, dim3(SCAN_THREADS), 0, stream, true,         \
                  (const float*)q, (const float*)k, (const float*)v, (const float*)coef,        \
                  (const float*)kq, (const T*)projected, state, slots, request_start, o, sizes, \
                  write)
    if (D <= 16) SCAN(4);
    else if (D <= 32) SCAN(8);
    else if (D <= 64) SCAN(16);
    else if (D <= 128) SCAN(32);
    else SCAN(64);
#undef SCAN
    MLXONE_LAUNCH_CHECK("gated delta rule (scan)");
    const long long items = (long long)tokens * H;
    launch_kernel(delta_finish_kernel<T>, dim3(ceil_div_host(items, 8)), dim3(256), 0, stream, true,
                  (const float*)o, (const T*)projected, norm_weight, (T*)mixed, items, sizes, eps);
    MLXONE_LAUNCH_CHECK("gated delta rule (finish)");
    return 0;
}

}  // namespace

// 32-bit values of scratch that a call with `tokens` tokens needs.
MLXONE_API long long mlxone_gated_delta_scratch(int tokens, int heads, int kv_heads, int key_dim,
                                                int value_dim) {
    return (long long)tokens * (2LL * kv_heads * key_dim + 2LL * heads * value_dim + 2LL * heads +
                                kv_heads);
}

// 32-bit values of a request's slot.
MLXONE_API long long mlxone_gated_delta_state(int heads, int kv_heads, int key_dim, int value_dim,
                                              int taps) {
    const DeltaSizes sizes = {heads, kv_heads, key_dim, value_dim, taps};
    return sizes.state();
}

MLXONE_API int mlxone_gated_delta(const void* projected, const float* conv, const float* a_log,
                                  const float* dt_bias, const float* norm_weight, float eps,
                                  float unit_eps, float* state, const int* slots,
                                  const int* token_request, const int* request_start,
                                  const int* history, float* scratch, void* mixed, int tokens,
                                  int requests, int heads, int kv_heads, int key_dim, int value_dim,
                                  int taps, int write, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && requests > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                   "gated delta rule: bad sizes");
    MLXONE_REQUIRE(key_dim >= 1 && key_dim <= 256, "gated delta rule: key size %d is not in 1..256",
                   key_dim);
    MLXONE_REQUIRE(value_dim >= 1 && taps >= 1, "gated delta rule: bad value size or taps");
    MLXONE_REQUIRE(requests <= 65535 && heads < 65535, "gated delta rule: too many requests or heads");
    const DeltaSizes sizes = {heads, kv_heads, key_dim, value_dim, taps};
    if (dtype == MLXONE_BF16)
        return launch_delta<__nv_bfloat16>(projected, conv, a_log, dt_bias, norm_weight, eps,
                                           unit_eps, state, slots, token_request, request_start,
                                           history, scratch, mixed, tokens, requests, sizes, write,
                                           stream);
    return launch_delta<float>(projected, conv, a_log, dt_bias, norm_weight, eps, unit_eps, state,
                               slots, token_request, request_start, history, scratch, mixed, tokens,
                               requests, sizes, write, stream);
}
