// Operations on the 32-bit residual stream and on activations that have no product in them:
// vectors added before a pass of a loop, activations of a dense feed-forward, and the mean of
// several mixers' outputs, each divided by its root mean square.
#include "common.cuh"

// ------------------------------------------------------------------ add vectors
// residual[t, :] += delta[t, :] (if delta) + table[ids[t], :] (if table) + vector[:] (if vector).
template <typename T>
__global__ void add_vectors_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const int* __restrict__ ids, const T* __restrict__ table,
                                   const float* __restrict__ vector, int hidden, int vocab) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const T* row = nullptr;
    if (table != nullptr) {
        int id = ids[t];
        id = min(max(id, 0), vocab - 1);          // (the embedding kernel has reported a bad id)
        row = table + (size_t)id * hidden;
    }
    float* dst = residual + (size_t)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = dst[c];
        if (delta != nullptr) v += to_float<T>(delta[(size_t)t * hidden + c]);
        if (row != nullptr) v += to_float<T>(row[c]);
        if (vector != nullptr) v += vector[c];
        dst[c] = v;
    }
}

MLXONE_API int mlxone_add_vectors(float* residual, const void* delta, const int* ids,
                                  const void* table, const float* vector, int tokens, int hidden,
                                  int vocab, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0, "add_vectors: bad sizes");
    MLXONE_REQUIRE(table == nullptr || (ids != nullptr && vocab > 0), "add_vectors: a table needs ids");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16)
        launch_kernel(add_vectors_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, true,
                      residual, (const __nv_bfloat16*)delta, ids, (const __nv_bfloat16*)table, vector,
                      hidden, vocab);
    else
        launch_kernel(add_vectors_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                      residual, (const float*)delta, ids, (const float*)table, vector, hidden, vocab);
    MLXONE_LAUNCH_CHECK("add_vectors");
    return 0;
}

// ------------------------------------------------------------------ activations
enum : int { ACT_RELU2 = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_RELU = 3 };

__device__ __forceinline__ float activate(float z, int kind) {
    switch (kind) {
        case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
        case ACT_GELU_TANH:
            return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        case ACT_SILU: return z / (1.f + expf(-z));
        default: return fmaxf(z, 0.f);
    }
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, long long total,
                                  int kind) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_float<T>(activate(to_float<T>(x[i]), kind));
}

// bfloat16, eight values a thread
__global__ void activation_wide_kernel(const __nv_bfloat16* __restrict__ x,
                                       __nv_bfloat16* __restrict__ out, long long groups, int kind) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + i * 8);
    const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 packed;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int k = 0; k < 4; ++k)
        q[k] = __floats2bfloat162_rn(activate(__low2float(in[k]), kind),
                                     activate(__high2float(in[k]), kind));
    *reinterpret_cast<uint4*>(out + i * 8) = packed;
}

MLXONE_API int mlxone_activation(const void* x, void* out, long long total, int kind, int dtype,
                                 cudaStream_t stream) {
    if (total == 0) return 0;
    MLXONE_REQUIRE(total > 0 && kind >= 0 && kind <= 3, "activation: bad arguments");
    if (dtype == MLXONE_BF16 && total % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0)
        launch_kernel(activation_wide_kernel, dim3(ceil_div_host(total / 8, 256)), dim3(256), 0,
                      stream, true, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, total / 8, kind);
    else if (dtype == MLXONE_BF16)
        launch_kernel(activation_kernel<__nv_bfloat16>, dim3(ceil_div_host(total, 256)), dim3(256), 0,
                      stream, true, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, total, kind);
    else
        launch_kernel(activation_kernel<float>, dim3(ceil_div_host(total, 256)), dim3(256), 0, stream,
                      true, (const float*)x, (float*)out, total, kind);
    MLXONE_LAUNCH_CHECK("activation");
    return 0;
}

// ------------------------------------------------------------------ mean of normed branches
// residual[t, :] += (1 / n) * sum_b x_b[t, :] * rsqrt(mean(x_b[t, :]^2) + eps) * weight_b[:],
// for n <= 4 branches, all in 32-bit. One block per token; the sums of squares are added in an
// order that the row length fixes.
constexpr int MAX_BRANCHES = 4;

template <typename T>
struct Branches {
    const T* x[MAX_BRANCHES];
    const float* weight[MAX_BRANCHES];
};

template <typename T>
__global__ void normed_mean_add_kernel(float* __restrict__ residual, Branches<T> branches, int count,
                                       int hidden, float eps) {
    __shared__ float scratch[33];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    float inv[MAX_BRANCHES];
#pragma unroll
    for (int b = 0; b < MAX_BRANCHES; ++b) {
        inv[b] = 0.f;
        if (b >= count) continue;
        const T* row = branches.x[b] + (size_t)t * hidden;
        float sum = 0.f;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = to_float<T>(row[c]);
            sum = fmaf(v, v, sum);
        }
        sum = block_sum(sum, scratch);
        inv[b] = rsqrtf(sum / (float)hidden + eps);
    }
    const float share = 1.f / (float)count;
    float* dst = residual + (size_t)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float total = 0.f;
#pragma unroll
        for (int b = 0; b < MAX_BRANCHES; ++b)
            if (b < count)
                total += to_float<T>(branches.x[b][(size_t)t * hidden + c]) * inv[b] *
                         branches.weight[b][c];
        dst[c] += total * share;
    }
}

MLXONE_API int mlxone_normed_mean_add(float* residual, const void* const* x,
                                      const float* const* weight, int count, int tokens, int hidden,
                                      float eps, int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(count >= 1 && count <= MAX_BRANCHES, "normed_mean_add: 1 to %d branches, got %d",
                   MAX_BRANCHES, count);
    MLXONE_REQUIRE(tokens > 0 && hidden > 0, "normed_mean_add: bad sizes");
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (dtype == MLXONE_BF16) {
        Branches<__nv_bfloat16> b = {};
        for (int i = 0; i < count; ++i) { b.x[i] = (const __nv_bfloat16*)x[i]; b.weight[i] = weight[i]; }
        launch_kernel(normed_mean_add_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                      true, residual, b, count, hidden, eps);
    } else {
        Branches<float> b = {};
        for (int i = 0; i < count; ++i) { b.x[i] = (const float*)x[i]; b.weight[i] = weight[i]; }
        launch_kernel(normed_mean_add_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                      residual, b, count, hidden, eps);
    }
    MLXONE_LAUNCH_CHECK("normed_mean_add");
    return 0;
}
