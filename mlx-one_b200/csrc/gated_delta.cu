// The gated delta rule over a ragged batch, with per-request state in 32-bit slots.
//
// projected[t] (rows `ld` values apart: it may be a slice of a wider product) =
// [q: G x D | k: G x D | v: H x V | gate: H x V | beta: H | decay: H] (G query/key
// heads of D values, H value heads of V values; value head h reads query/key head h / (H / G)).
// The first C = 2 G D + H V channels pass a causal convolution over the last `taps` tokens of the
// request (conv [C, taps], last column the current token's) and silu.
//
// A request's slot holds, in 32-bit: S [H, D, V], then a ring of the convolution's inputs
// [taps, C]: row p % taps is the input at position p. A step writes the rows of its own
// positions and reads the taps - 1 rows before them, which are never the same rows, so that
// writers and readers of one step need no order among themselves.
//
// A step with portions runs three kernels:
//   prepare  per token: convolution + silu; q and k to unit length per head (q also times
//            D^-1/2); beta = sigmoid, g = exp(-exp(A_log) softplus(a + dt_bias)); k.q per head.
//   scan     per (request, value head, tile of columns of S): for each token of the request, in
//            order:  S = g S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q.
//            A column of S depends on no other column, so columns are spread over threads and
//            blocks; a column's D values are spread over eight lanes of a warp. With the dot
//            products of the column with k and q taken before the update,
//            u = beta (v - g (S.k)) and o = g (S.q) + u (k.q). Four tokens are worked on
//            together: one pass takes the sums of the column, as it stands before the four,
//            with their k and q; with the products k_i.k_j and k_i.q_j of the four (worked out
//            once per block) the four u and o follow from numbers alone; a second pass updates
//            the column for all four. The operands of the next 16 tokens travel to shared
//            memory (cp.async) while the current 16 are worked on. Extra blocks write the
//            convolution's inputs into the ring.
//   finish   per (token, head): o / rms(o) * weight * silu(gate), in the compute type.
// A step of single tokens runs one kernel, a block per (request, value head): the head's
// matrix is asked for before the wait for the projection, the convolutions, norms and gates of
// its own channels are worked out in the block, the recurrence takes one pass, and the output's
// norm and gate follow after a reduction over the block.
#include "common.cuh"

namespace {

constexpr int PREP_THREADS = 256;
constexpr int SCAN_THREADS = 128;
constexpr int CHUNK = 16;            // tokens whose operands are staged in shared memory together
constexpr int STEP_LANES = 4;        // single-token kernel: lanes that share a column of S
constexpr int STEP_MAX_COLUMNS = 128;

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ void copy_async_4(float* dst, const float* src) {
    const uint32_t to = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(to), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_async_16(float* dst, const float* src) {
    const uint32_t to = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(src) : "memory");
}
template <int N>
__device__ __forceinline__ void copy_wait_for() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct DeltaSizes {
    int heads, kv_heads, key_dim, value_dim, taps;
    __host__ __device__ int qk() const { return kv_heads * key_dim; }
    __host__ __device__ int inner() const { return heads * value_dim; }
    __host__ __device__ int channels() const { return 2 * qk() + inner(); }
    __host__ __device__ int width() const { return channels() + inner() + 2 * heads; }
    __host__ __device__ long long matrices() const { return (long long)heads * key_dim * value_dim; }
    __host__ __device__ long long state() const {
        return matrices() + (long long)taps * channels();
    }
};

// The input of channel c at `position` - back, for a token at place `index` of its portion:
// a row of this step, the ring, or zero before the request's start.
template <typename T>
__device__ __forceinline__ float conv_input(const T* projected, int ld, const float* ring,
                                            int channels, int taps, int t, int index, int position,
                                            int back, int c) {
    if (index - back >= 0) return to_float<T>(projected[(size_t)(t - back) * ld + c]);
    if (position - back >= 0) return ring[(size_t)((position - back) % taps) * channels + c];
    return 0.f;
}

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
                     float* __restrict__ kq, DeltaSizes sizes, float unit_eps, int ld) {
    extern __shared__ float mixed[];                 // the token's C channels after conv + silu
    griddep_wait();
    const int t = blockIdx.x;
    const int r = token_request[t];
    const int index = t - request_start[r];
    const int position = history[r] + index;
    const int taps = sizes.taps, channels = sizes.channels(), width = ld;
    const float* ring = state + (size_t)slots[r] * sizes.state() + sizes.matrices();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = 0.f;
        for (int j = 0; j < taps; ++j)
            y = fmaf(conv[(size_t)c * taps + j],
                     conv_input<T>(projected, ld, ring, channels, taps, t, index, position,
                                   taps - 1 - j, c), y);
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
    // (the scan's blocks would only wait beside this kernel's if they were let in earlier)
    griddep_launch();
}

// ------------------------------------------------------------------ scan
// Grid (column tiles, H + 1, requests); blocks with blockIdx.y == H write the convolution's
// inputs into the ring. A thread keeps PER values of its column: element e of lane l is row
// (e / 4) * 4 LANES + l * 4 + e % 4 of S, so that the lanes read k and q as neighbouring float4.
// Dynamic shared memory: two buffers of [CHUNK][ROWS] for k and for q, [CHUNK][COLUMNS] for v and
// [CHUNK] for each of g, beta and k.q.
template <typename T, int PER, int LANES>
__global__ void __launch_bounds__(SCAN_THREADS)
delta_scan_kernel(const float* __restrict__ q_in, const float* __restrict__ k_in,
                  const float* __restrict__ v_in, const float* __restrict__ coef,
                  const float* __restrict__ kq, const T* __restrict__ projected,
                  float* __restrict__ state, const int* __restrict__ slots,
                  const int* __restrict__ request_start, const int* __restrict__ history,
                  float* __restrict__ out, DeltaSizes sizes, int write, int ld) {
    constexpr int ROWS = PER * LANES;                 // rows of S a thread group covers (>= D)
    constexpr int COLUMNS = SCAN_THREADS / LANES;     // columns of S per block
    constexpr int BUFFER = CHUNK * (2 * ROWS + COLUMNS + 3);
    constexpr int GROUP = 4;                          // tokens worked on together
    extern __shared__ __align__(16) float staged[];
    __shared__ float gram[CHUNK / GROUP][2][GROUP][GROUP];   // k_i.k_t and k_i.q_t, i < t in a group
    griddep_wait();
    const int r = blockIdx.z;
    const int first = request_start[r], last = request_start[r + 1];
    const int H = sizes.heads, G = sizes.kv_heads, D = sizes.key_dim, V = sizes.value_dim;
    float* slot = state + (size_t)slots[r] * sizes.state();
    if (blockIdx.y == H) {
        // the inputs of the portion's last positions (at most taps of them) go into the ring
        griddep_launch();
        if (!write) return;
        const int channels = sizes.channels(), taps = sizes.taps;
        const int n = last - first, kept = min(n, taps);
        float* ring = slot + sizes.matrices();
        for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels;
             c += gridDim.x * blockDim.x)
            for (int index = n - kept; index < n; ++index)
                ring[(size_t)((history[r] + index) % taps) * channels + c] =
                    to_float<T>(projected[(size_t)(first + index) * ld + c]);
        return;
    }
    const int h = blockIdx.y, g = h / (H / G);
    const int lane = threadIdx.x & (LANES - 1);
    const int local = threadIdx.x / LANES;
    const int column = blockIdx.x * COLUMNS + local;
    const bool live = column < V;
    float* matrix = slot + (size_t)h * D * V;
    float S[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int row = (e / 4) * (4 * LANES) + lane * 4 + e % 4;
        S[e] = live && row < D ? matrix[(size_t)row * V + column] : 0.f;
    }
    // whether k, q and v rows can travel 16 bytes at a time
    const bool quads = D % 4 == 0 && V % 4 == 0 &&
                       ((reinterpret_cast<uintptr_t>(q_in) | reinterpret_cast<uintptr_t>(k_in) |
                         reinterpret_cast<uintptr_t>(v_in)) & 15) == 0;
    // rows behind D and columns behind V stay zero in both buffers
    for (int i = threadIdx.x; i < 2 * BUFFER; i += SCAN_THREADS) staged[i] = 0.f;
    __syncthreads();
    auto fetch = [&](int base, int buffer) {
        const int count = min(CHUNK, last - base);
        float* ks = staged + buffer * BUFFER;
        float* qs = ks + CHUNK * ROWS;
        float* vs = qs + CHUNK * ROWS;
        float* cs = vs + CHUNK * COLUMNS;
        const int wide = min(COLUMNS, V - (int)blockIdx.x * COLUMNS);
        if (quads) {
            // rows of a multiple of four values: 16 bytes a copy
            const int per_row = D / 4;
            const bool power = (per_row & (per_row - 1)) == 0;
            const int shift = __ffs(per_row) - 1;
            for (int i = threadIdx.x; i < count * per_row; i += SCAN_THREADS) {
                const int t = power ? i >> shift : i / per_row;
                const int e = (i - t * per_row) * 4;
                const size_t at = ((size_t)(base + t) * G + g) * D + e;
                copy_async_16(ks + t * ROWS + e, k_in + at);
                copy_async_16(qs + t * ROWS + e, q_in + at);
            }
            for (int i = threadIdx.x; i < count * (wide / 4); i += SCAN_THREADS) {
                const int t = i / (wide / 4), c = (i % (wide / 4)) * 4;
                copy_async_16(vs + t * COLUMNS + c,
                              v_in + ((size_t)(base + t) * H + h) * V + blockIdx.x * COLUMNS + c);
            }
        } else {
            for (int i = threadIdx.x; i < count * D; i += SCAN_THREADS) {
                const int t = i / D, e = i % D;
                const size_t at = ((size_t)(base + t) * G + g) * D + e;
                copy_async_4(ks + t * ROWS + e, k_in + at);
                copy_async_4(qs + t * ROWS + e, q_in + at);
            }
            for (int i = threadIdx.x; i < count * wide; i += SCAN_THREADS) {
                const int t = i / wide, c = i % wide;
                copy_async_4(vs + t * COLUMNS + c,
                             v_in + ((size_t)(base + t) * H + h) * V + blockIdx.x * COLUMNS + c);
            }
        }
        if (threadIdx.x < count) {
            const size_t at = (size_t)(base + threadIdx.x) * H + h;
            copy_async_4(cs + threadIdx.x, coef + at * 2);
            copy_async_4(cs + CHUNK + threadIdx.x, coef + at * 2 + 1);
            copy_async_4(cs + 2 * CHUNK + threadIdx.x, kq + (size_t)(base + threadIdx.x) * G + g);
        } else if (threadIdx.x < CHUNK) {
            // places behind the portion's end: a token that changes nothing (g = 1, beta = 0)
            cs[threadIdx.x] = 1.f;
            cs[CHUNK + threadIdx.x] = 0.f;
            cs[2 * CHUNK + threadIdx.x] = 0.f;
        }
        copy_commit();
    };
    if (first < last) fetch(first, 0);
    int buffer = 0;
    for (int base = first; base < last; base += CHUNK, buffer ^= 1) {
        const int count = min(CHUNK, last - base);
        if (base + CHUNK < last) {
            fetch(base + CHUNK, buffer ^ 1);
            copy_wait_for<1>();
        } else {
            copy_wait_for<0>();
        }
        __syncthreads();
        const float* ks = staged + buffer * BUFFER;
        const float* qs = ks + CHUNK * ROWS;
        const float* vs = qs + CHUNK * ROWS;
        const float* cs = vs + CHUNK * COLUMNS;
        // the products k_i.k_t and k_i.q_t of the pairs i < t inside each group of four tokens:
        // 4 groups x 6 pairs x 2 kinds, each by LANES lanes
        for (int item = threadIdx.x / LANES; item < (CHUNK / GROUP) * 12; item += SCAN_THREADS / LANES) {
            const int group = item / 12, kind = (item % 12) / 6, pair = item % 6;
            const int t = pair < 1 ? 1 : (pair < 3 ? 2 : 3);
            const int i = pair - (t == 1 ? 0 : (t == 2 ? 1 : 3));
            const float* left = ks + (group * GROUP + i) * ROWS;
            const float* right = (kind ? qs : ks) + (group * GROUP + t) * ROWS;
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < PER; e += 4) {
                const int at = (e / 4) * (4 * LANES) + lane * 4;
                const float4 x = *reinterpret_cast<const float4*>(left + at);
                const float4 y = *reinterpret_cast<const float4*>(right + at);
                dot = fmaf(x.x, y.x, dot); dot = fmaf(x.y, y.y, dot);
                dot = fmaf(x.z, y.z, dot); dot = fmaf(x.w, y.w, dot);
            }
#pragma unroll
            for (int across = 1; across < LANES; across <<= 1)
                dot += __shfl_xor_sync(0xffffffffu, dot, across);
            if (lane == 0) gram[group][kind][i][t] = dot;
        }
        __syncthreads();
        for (int t0 = 0; t0 < count; t0 += GROUP) {
            // the sums of this column (as it stands before the group) with the four k and q
            float a[GROUP] = {0.f, 0.f, 0.f, 0.f}, b[GROUP] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < PER; e += 4) {
                const int at = (e / 4) * (4 * LANES) + lane * 4;
#pragma unroll
                for (int j = 0; j < GROUP; ++j) {
                    const float4 k4 = *reinterpret_cast<const float4*>(ks + (t0 + j) * ROWS + at);
                    const float4 q4 = *reinterpret_cast<const float4*>(qs + (t0 + j) * ROWS + at);
                    a[j] = fmaf(S[e], k4.x, a[j]); b[j] = fmaf(S[e], q4.x, b[j]);
                    a[j] = fmaf(S[e + 1], k4.y, a[j]); b[j] = fmaf(S[e + 1], q4.y, b[j]);
                    a[j] = fmaf(S[e + 2], k4.z, a[j]); b[j] = fmaf(S[e + 2], q4.z, b[j]);
                    a[j] = fmaf(S[e + 3], k4.w, a[j]); b[j] = fmaf(S[e + 3], q4.w, b[j]);
                }
            }
#pragma unroll
            for (int across = 1; across < LANES; across <<= 1) {
#pragma unroll
                for (int j = 0; j < GROUP; ++j) {
                    a[j] += __shfl_xor_sync(0xffffffffu, a[j], across);
                    b[j] += __shfl_xor_sync(0xffffffffu, b[j], across);
                }
            }
            // token by token with numbers only. With s_j the column after token j of the group and
            // c(i, j) = g_(i+1) ... g_(j-1):  s_(j-1).x = g_1 .. g_(j-1) (s_0.x) + sum_(i<j) c(i, j) (k_i.x) u_i
            const int group = t0 / GROUP;
            float decay[GROUP], u[GROUP];
#pragma unroll
            for (int j = 0; j < GROUP; ++j) decay[j] = cs[t0 + j];
            float before = 1.f;                       // g_1 ... g_(j-1)
#pragma unroll
            for (int j = 0; j < GROUP; ++j) {
                float with_k = before * a[j], with_q = before * b[j];
                float carry = 1.f;                    // c(i, j), from i = j - 1 downwards
#pragma unroll
                for (int i = j - 1; i >= 0; --i) {
                    with_k = fmaf(carry * gram[group][0][i][j], u[i], with_k);
                    with_q = fmaf(carry * gram[group][1][i][j], u[i], with_q);
                    carry *= decay[i];
                }
                u[j] = cs[CHUNK + t0 + j] * (vs[(t0 + j) * COLUMNS + local] - decay[j] * with_k);
                if (live && lane == 0 && t0 + j < count)
                    out[((size_t)(base + t0 + j) * H + h) * V + column] =
                        fmaf(u[j], cs[2 * CHUNK + t0 + j], decay[j] * with_q);
                before *= decay[j];
            }
            // s_4 = g_1 .. g_4 s_0 + sum_i (g_(i+1) .. g_4) k_i u_i
            float weight[GROUP];
            float after = 1.f;
#pragma unroll
            for (int j = GROUP - 1; j >= 0; --j) {
                weight[j] = u[j] * after;
                after *= decay[j];
            }
#pragma unroll
            for (int e = 0; e < PER; e += 4) {
                const int at = (e / 4) * (4 * LANES) + lane * 4;
                float next[4] = {after * S[e], after * S[e + 1], after * S[e + 2], after * S[e + 3]};
#pragma unroll
                for (int j = 0; j < GROUP; ++j) {
                    const float4 k4 = *reinterpret_cast<const float4*>(ks + (t0 + j) * ROWS + at);
                    next[0] = fmaf(k4.x, weight[j], next[0]);
                    next[1] = fmaf(k4.y, weight[j], next[1]);
                    next[2] = fmaf(k4.z, weight[j], next[2]);
                    next[3] = fmaf(k4.w, weight[j], next[3]);
                }
                S[e] = next[0]; S[e + 1] = next[1]; S[e + 2] = next[2]; S[e + 3] = next[3];
            }
        }
        __syncthreads();          // the buffer is fetched into again two rounds on
    }
    // the kernels behind this one may start now: earlier they would sit on the SMs beside a
    // kernel that runs long on few warps
    griddep_launch();
    if (write && live) {
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int row = (e / 4) * (4 * LANES) + lane * 4 + e % 4;
            if (row < D) matrix[(size_t)row * V + column] = S[e];
        }
    }
}

// ------------------------------------------------------------------ a step of single tokens
// One block per (value head, request); request r brings token r. Threads: STEP_LANES per column
// of S. Dynamic shared memory: q and k [ROWS each], v and o [V each], four scalars.
template <typename T, int PER>
__global__ void __launch_bounds__(STEP_LANES * STEP_MAX_COLUMNS)
delta_step_kernel(const T* __restrict__ projected, const float* __restrict__ conv,
                  const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                  const float* __restrict__ norm_weight, float eps, float unit_eps,
                  float* __restrict__ state, const int* __restrict__ slots,
                  const int* __restrict__ history, T* __restrict__ mixed, DeltaSizes sizes,
                  int write, int ld) {
    constexpr int LANES = STEP_LANES;
    constexpr int ROWS = PER * LANES;
    extern __shared__ __align__(16) float staged[];
    const int H = sizes.heads, G = sizes.kv_heads, D = sizes.key_dim, V = sizes.value_dim;
    const int taps = sizes.taps, channels = sizes.channels();
    float* qs = staged;
    float* ks = qs + ROWS;
    float* vs = ks + ROWS;
    float* os = vs + V;
    float* scalars = os + V;                 // k.q, decay, beta, 1 / rms(o)
    griddep_launch();
    const int h = blockIdx.x, r = blockIdx.y, g = h / (H / G);
    const int lane = threadIdx.x & (LANES - 1), column = threadIdx.x / LANES;
    const bool live = column < V;
    // the head's matrix was written by an earlier step: its loads start before the wait for
    // the kernel that writes this step's projection
    float* slot = state + (size_t)slots[r] * sizes.state();
    float* matrix = slot + (size_t)h * D * V;
    float S[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int row = (e / 4) * (4 * LANES) + lane * 4 + e % 4;
        S[e] = live && row < D ? matrix[(size_t)row * V + column] : 0.f;
    }
    for (int i = threadIdx.x; i < 2 * ROWS; i += blockDim.x) qs[i] = 0.f;      // q and k, padded
    __syncthreads();
    griddep_wait();
    const int t = r, position = history[r];
    float* ring = slot + sizes.matrices();
    const T* row_in = projected + (size_t)t * ld;
    // convolution + silu of this block's channels: its key head's q and k, its own v
    const bool owner = h % (H / G) == 0;         // writes the key head's inputs into the ring
    for (int i = threadIdx.x; i < 2 * D + V; i += blockDim.x) {
        const int c = i < D ? g * D + i : (i < 2 * D ? sizes.qk() + g * D + (i - D)
                                                     : 2 * sizes.qk() + h * V + (i - 2 * D));
        const float now = to_float<T>(row_in[c]);
        float y = conv[(size_t)c * taps + taps - 1] * now;
        for (int j = 0; j + 1 < taps; ++j) {
            const int before = position - (taps - 1 - j);
            if (before >= 0)
                y = fmaf(conv[(size_t)c * taps + j], ring[(size_t)(before % taps) * channels + c], y);
        }
        if (write && (i >= 2 * D || owner)) ring[(size_t)(position % taps) * channels + c] = now;
        const float value = silu(y);
        if (i < D) qs[i] = value;
        else if (i < 2 * D) ks[i - D] = value;
        else vs[i - 2 * D] = value;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, in_warp = threadIdx.x & 31;
    if (warp == 0) {
        float qq = 0.f, kk = 0.f;
        for (int e = in_warp; e < D; e += 32) {
            qq = fmaf(qs[e], qs[e], qq);
            kk = fmaf(ks[e], ks[e], kk);
        }
        qq = warp_sum(qq);
        kk = warp_sum(kk);
        const float q_scale = rsqrtf((float)D) / sqrtf(qq + unit_eps);
        const float k_scale = 1.f / sqrtf(kk + unit_eps);
        float dot = 0.f;
        for (int e = in_warp; e < D; e += 32) {
            const float qv = qs[e] * q_scale, kv = ks[e] * k_scale;
            qs[e] = qv;
            ks[e] = kv;
            dot = fmaf(qv, kv, dot);
        }
        dot = warp_sum(dot);
        if (in_warp == 0) {
            scalars[0] = dot;
            const T* tail = row_in + channels + sizes.inner();
            scalars[1] = expf(-expf(a_log[h]) * softplus(to_float<T>(tail[H + h]) + dt_bias[h]));
            scalars[2] = 1.f / (1.f + expf(-to_float<T>(tail[h])));
        }
    }
    __syncthreads();
    {
        float k[PER];
        float wk[4] = {0.f, 0.f, 0.f, 0.f}, wq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < PER; e += 4) {
            const int at = (e / 4) * (4 * LANES) + lane * 4;
            const float4 k4 = *reinterpret_cast<const float4*>(ks + at);
            const float4 q4 = *reinterpret_cast<const float4*>(qs + at);
            k[e] = k4.x; k[e + 1] = k4.y; k[e + 2] = k4.z; k[e + 3] = k4.w;
            wk[0] = fmaf(S[e], k4.x, wk[0]); wq[0] = fmaf(S[e], q4.x, wq[0]);
            wk[1] = fmaf(S[e + 1], k4.y, wk[1]); wq[1] = fmaf(S[e + 1], q4.y, wq[1]);
            wk[2] = fmaf(S[e + 2], k4.z, wk[2]); wq[2] = fmaf(S[e + 2], q4.z, wq[2]);
            wk[3] = fmaf(S[e + 3], k4.w, wk[3]); wq[3] = fmaf(S[e + 3], q4.w, wq[3]);
        }
        float with_k = (wk[0] + wk[1]) + (wk[2] + wk[3]);
        float with_q = (wq[0] + wq[1]) + (wq[2] + wq[3]);
#pragma unroll
        for (int across = 1; across < LANES; across <<= 1) {
            with_k += __shfl_xor_sync(0xffffffffu, with_k, across);
            with_q += __shfl_xor_sync(0xffffffffu, with_q, across);
        }
        const float decay = scalars[1];
        const float u = scalars[2] * ((live ? vs[column] : 0.f) - decay * with_k);
        if (write && live) {
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                const int row = (e / 4) * (4 * LANES) + lane * 4 + e % 4;
                if (row < D) matrix[(size_t)row * V + column] = fmaf(k[e], u, decay * S[e]);
            }
        }
        if (live && lane == 0) os[column] = fmaf(u, scalars[0], decay * with_q);
    }
    __syncthreads();
    if (warp == 0) {
        float sum = 0.f;
        for (int e = in_warp; e < V; e += 32) sum = fmaf(os[e], os[e], sum);
        sum = warp_sum(sum);
        if (in_warp == 0) scalars[3] = 1.f / sqrtf(sum / (float)V + eps);
    }
    __syncthreads();
    const T* gate = row_in + channels + (size_t)h * V;
    for (int e = threadIdx.x; e < V; e += blockDim.x)
        mixed[(size_t)t * sizes.inner() + (size_t)h * V + e] =
            from_float<T>(os[e] * scalars[3] * norm_weight[e] * silu(to_float<T>(gate[e])));
}

// ------------------------------------------------------------------ finish
// One warp per (token, head): mixed[t, h, :] = o / sqrt(mean(o^2) + eps) * weight * silu(gate).
template <typename T>
__global__ void __launch_bounds__(256)
delta_finish_kernel(const float* __restrict__ o, const T* __restrict__ projected,
                    const float* __restrict__ weight, T* __restrict__ mixed, long long items,
                    DeltaSizes sizes, float eps, int ld) {
    griddep_launch();
    griddep_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const int H = sizes.heads, V = sizes.value_dim;
    const long long t = item / H;
    const int h = (int)(item % H);
    const float* row = o + item * V;
    const T* gate = projected + (size_t)t * ld + sizes.channels() + (size_t)h * V;
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
                 DeltaSizes sizes, int write, int ld, int single, cudaStream_t stream) {
    const int G = sizes.kv_heads, D = sizes.key_dim, H = sizes.heads, V = sizes.value_dim;
    if (single && tokens == requests && V <= STEP_MAX_COLUMNS) {
        // every request brings one token: one kernel
        const int per = D <= 16 ? 4 : D <= 32 ? 8 : D <= 64 ? 16 : D <= 128 ? 32 : 64;
        const size_t shared = (size_t)(2 * per * STEP_LANES + 2 * V + 4) * sizeof(float);
        const int threads = (STEP_LANES * V + 31) / 32 * 32;
#define STEP(PER)                                                                              \
    launch_kernel(delta_step_kernel<T, PER>, dim3(H, requests), dim3(threads), shared, stream, \
                  true, (const T*)projected, conv, a_log, dt_bias, norm_weight, eps, unit_eps, \
                  state, slots, history, (T*)mixed, sizes, write, ld)
        if (per == 4) STEP(4);
        else if (per == 8) STEP(8);
        else if (per == 16) STEP(16);
        else if (per == 32) STEP(32);
        else STEP(64);
#undef STEP
        MLXONE_LAUNCH_CHECK("gated delta rule (single tokens)");
        return 0;
    }
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
                  token_request, request_start, history, q, k, v, coef, kq, sizes, unit_eps, ld);
    MLXONE_LAUNCH_CHECK("gated delta rule (prepare)");
    // A column's values are spread over 8 lanes (16 for keys longer than 128). Measured at 16 heads
    // of 128 x 128 and 2048 tokens: with 16 lanes every lane repeats the four tokens' solve for
    // half as many values of its own, 292 M warp instructions and 702 us.
#define SCAN(PER, LANES)                                                                          \
    do {                                                                                          \
        constexpr int COLUMNS = SCAN_THREADS / LANES;                                             \
        const dim3 grid(ceil_div_host(V, COLUMNS), H + 1, requests);                              \
        const size_t staged = (size_t)2 * CHUNK * (2 * PER * LANES + COLUMNS + 3) * sizeof(float); \
        if (staged > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(delta_scan_kernel<T, PER, LANES>,                                \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staged);       \
        launch_kernel(delta_scan_kernel<T, PER, LANES>, grid, dim3(SCAN_THREADS), staged, stream, \
                      true, (const float*)q, (const float*)k, (const float*)v,                    \
                      (const float*)coef, (const float*)kq, (const T*)projected, state, slots,    \
                      request_start, history, o, sizes, write, ld);                               \
    } while (0)
    // ... with 8 lanes 156 M instructions and 536 us. (16 lanes only where a grid of 8-lane blocks
    // would leave half the SMs empty was measured too, 8 heads: 1112 us against 947 us.)
    if (D <= 32) SCAN(4, 8);
    else if (D <= 64) SCAN(8, 8);
    else if (D <= 128) SCAN(16, 8);
    else SCAN(16, 16);
#undef SCAN
    MLXONE_LAUNCH_CHECK("gated delta rule (scan)");
    const long long items = (long long)tokens * H;
    launch_kernel(delta_finish_kernel<T>, dim3(ceil_div_host(items, 8)), dim3(256), 0, stream, true,
                  (const float*)o, (const T*)projected, norm_weight, (T*)mixed, items, sizes, eps, ld);
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
                                  int taps, int write, int ld, int single, int dtype,
                                  cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && requests > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                   "gated delta rule: bad sizes");
    MLXONE_REQUIRE(key_dim >= 1 && key_dim <= 256, "gated delta rule: key size %d is not in 1..256",
                   key_dim);
    MLXONE_REQUIRE(value_dim >= 1 && taps >= 1, "gated delta rule: bad value size or taps");
    MLXONE_REQUIRE(requests <= 65535 && heads < 65535, "gated delta rule: too many requests or heads");
    const DeltaSizes sizes = {heads, kv_heads, key_dim, value_dim, taps};
    MLXONE_REQUIRE(ld >= sizes.width(), "gated delta rule: rows %d apart are shorter than %d", ld,
                   sizes.width());
    if (dtype == MLXONE_BF16)
        return launch_delta<__nv_bfloat16>(projected, conv, a_log, dt_bias, norm_weight, eps,
                                           unit_eps, state, slots, token_request, request_start,
                                           history, scratch, mixed, tokens, requests, sizes, write,
                                           ld, single, stream);
    return launch_delta<float>(projected, conv, a_log, dt_bias, norm_weight, eps, unit_eps, state,
                               slots, token_request, request_start, history, scratch, mixed, tokens,
                               requests, sizes, write, ld, single, stream);
}
