// Lightning attention: linear attention with a constant decay per head.
//
// Per token and head S = decay S + k v^T, o = S^T q, with q, k = silu of the projection's values
// [heads, D] and v likewise [heads, V]; S [D, V] is 32-bit and lives in the request's state slot
// ([heads][D][V]). The heads' outputs side by side are then divided by their common root mean
// square, multiplied by a weight and by sigmoid(gate), and stored in the compute dtype.
//
// A column of S depends on no other column. A block holds 32 columns of one head of one request:
// each of its four warps has all 32 columns and every fourth group of four rows of them in
// registers (a lane = a column, so the state moves 128 bytes at a time). The block walks the
// request's tokens of this step in order, eight at a time: the tokens' q and k (silu applied,
// 32-bit) and the block's slice of v are staged in shared memory, then every thread updates its
// part of the column and adds its share of o, and the four warps' shares meet in shared memory.
// Everything after the projection's silu is 32-bit.
//
// Long portions are cut into segments that run side by side (the recurrence is linear): every
// segment first builds, from a zero state, what its tokens add to the state; a short pass then
// chains the segments (S_in of a segment = decay^len of the one before, applied to its S_in, plus
// what that one added); finally every segment computes its outputs from its incoming state.
#include "common.cuh"

namespace {

constexpr int COLS = 32;          // columns of S per block
constexpr int LANES = 4;          // warps that share a column's rows
constexpr int THREADS = COLS * LANES;
constexpr int TOK = 8;            // tokens staged at a time

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }

struct ScanArgs {
    const void* projected;        // [tokens, ld]: q | k | v | gate
    int ld;
    const float* decay;           // [heads]
    float* state;                 // [slots][heads][D][V]
    const int* slots;             // [requests]
    const int* request_start;     // [requests + 1]
    float* o;                     // [tokens, heads * V] 32-bit outputs
    int heads, key_dim, value_dim;
    int write;
    // segments (null / 0: a request's tokens are one run from its state slot)
    int segment;                  // tokens per segment
    float* carried;               // [requests][segments][heads][D][V]
    int max_segments;
};

// MODE 0: from the slot through all tokens, outputs and the state written back (short portions
//         and single tokens).
// MODE 1: a segment from a zero state; its final state goes to `carried` (no outputs).
// MODE 2: a segment from its incoming state in `carried` (where the chaining pass has also put
//         the slot's state for segment 0, since the last segment's block overwrites the slot
//         while the first one's may not have started); outputs; the last segment writes the
//         slot. A request of one segment runs from its slot as in mode 0.
template <typename T, int DR, int MODE>
__global__ void __launch_bounds__(THREADS)
lightning_scan_kernel(ScanArgs a) {
    constexpr int DPAD = 4 * DR;                     // rows covered (>= key_dim)
    __shared__ __align__(16) float sq[TOK][DPAD];
    __shared__ __align__(16) float sk[TOK][DPAD];
    __shared__ float sv[TOK][COLS];
    __shared__ float parts[LANES][TOK][COLS];        // the warps' shares of the outputs
    // Within a group of eight tokens the state is kept divided by the decay's powers, so that
    // the recurrence costs one multiply-add per element and token instead of a multiply and a
    // multiply-add: token i's k is staged times decay^-(i+1), its q times decay^(i+1), and the
    // state is multiplied by decay^count after the group. Not for decays below 0.01, whose
    // inverse powers would leave the range of 32-bit numbers (they keep the plain form).
    __shared__ float kfac[TOK], qfac[TOK];
    griddep_launch();
    const int head = blockIdx.y;
    int request = blockIdx.z, piece = 0;
    if (MODE != 0) { request = blockIdx.z / a.max_segments; piece = blockIdx.z % a.max_segments; }
    // a warp holds 32 neighbouring columns (a row of S is read and written 128 bytes at a time);
    // the four warps share the rows: warp w keeps the groups of four rows w, w + 4, w + 8, ...
    const int col = threadIdx.x & 31, part = threadIdx.x >> 5;
    const int j = blockIdx.x * COLS + col;
    const int D = a.key_dim, V = a.value_dim, H = a.heads;
    const bool live = j < V;
    const float decay = a.decay[head];
    const bool scaled = decay >= 0.01f;
    if (threadIdx.x < TOK) {
        double power = 1.0;
        for (int i = 0; i <= (int)threadIdx.x; ++i) power *= (double)decay;
        qfac[threadIdx.x] = scaled ? (float)power : 1.f;
        kfac[threadIdx.x] = scaled ? (float)(1.0 / power) : 1.f;
    }
    float S[DR];
    if (MODE == 0) {
        // the state is what an earlier step left: it is asked for before the kernel ahead of
        // this one (the projection) is waited for, so that it comes while that one finishes
        const float* early = a.state + ((size_t)a.slots[request] * H + head) * (size_t)D * V;
#pragma unroll
        for (int m = 0; m < DR / 4; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = 4 * (part + LANES * m) + e;
                S[4 * m + e] = (live && row < D) ? early[(size_t)row * V + j] : 0.f;
            }
    }
    griddep_wait();
    int first = a.request_start[request];
    int last = a.request_start[request + 1];
    int pieces = 1;
    if (MODE != 0) {
        pieces = (last - first + a.segment - 1) / a.segment;
        if (piece >= pieces) return;
        if (MODE == 1 && piece == pieces - 1) return;      // nobody needs what the last one adds
        first += piece * a.segment;
        last = min(first + a.segment, last);
    }
    if (first >= last) return;
    const bool last_piece = MODE == 0 || last == a.request_start[request + 1];

    const size_t per_head = (size_t)D * V;
    float* slot = a.state + ((size_t)a.slots[request] * H + head) * per_head;
    float* carried = nullptr;
    if (MODE != 0)
        carried = a.carried + (((size_t)request * a.max_segments + piece) * H + head) * per_head;

    if (MODE != 0) {
        const float* from = MODE == 2 && pieces > 1 ? carried : slot;
#pragma unroll
        for (int m = 0; m < DR / 4; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = 4 * (part + LANES * m) + e;
                S[4 * m + e] = (MODE != 1 && live && row < D) ? from[(size_t)row * V + j] : 0.f;
            }
    }

    const T* projected = static_cast<const T*>(a.projected);
    const int q_at = head * D, k_at = H * D + head * D, v_at = 2 * H * D + head * V;
    // A thread's share of the staging of eight tokens: QN values of q and of k, VN of v. With
    // AHEAD their raw values for the next eight tokens are loaded into registers before the
    // current eight are multiplied, and become silu'd 32-bit numbers in shared memory afterwards.
    constexpr int QN = TOK * DPAD / THREADS, VN = TOK * COLS / THREADS;
    constexpr bool AHEAD = DR <= 32;
    float raw_q[AHEAD ? QN : 1], raw_k[AHEAD ? QN : 1], raw_v[AHEAD ? VN : 1];
    auto fetch = [&](int base, int count) {
#pragma unroll
        for (int i = 0; i < QN; ++i) {
            const int item = threadIdx.x + i * THREADS;
            const int t = item / DPAD, row = item % DPAD;
            raw_q[i] = raw_k[i] = 0.f;
            if (t < count && row < D) {
                const T* src = projected + (size_t)(base + t) * a.ld;
                if (MODE != 1) raw_q[i] = to_float<T>(src[q_at + row]);
                raw_k[i] = to_float<T>(src[k_at + row]);
            }
        }
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            const int item = threadIdx.x + i * THREADS;
            const int t = item / COLS, column = blockIdx.x * COLS + item % COLS;
            raw_v[i] = (t < count && column < V)
                ? to_float<T>(projected[(size_t)(base + t) * a.ld + v_at + column]) : 0.f;
        }
    };
    auto stash = [&](const bool whole, int count) {     // whole: all eight tokens are there
#pragma unroll
        for (int i = 0; i < QN; ++i) {
            const int item = threadIdx.x + i * THREADS;
            const int t = item / DPAD, row = item % DPAD;
            if (!whole && t >= count) continue;
            // (rows beyond the key size hold silu(0) = 0)
            sq[t][row] = MODE != 1 ? silu(raw_q[i]) * qfac[t] : 0.f;
            sk[t][row] = silu(raw_k[i]) * kfac[t];
        }
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            const int item = threadIdx.x + i * THREADS;
            if (whole || item / COLS < count) sv[item / COLS][item % COLS] = silu(raw_v[i]);
        }
    };
    if (AHEAD) fetch(first, min(TOK, last - first));
    for (int base = first; base < last; base += TOK) {
        const int count = min(TOK, last - base);
        __syncthreads();
        if (AHEAD) {
            if (count == TOK) stash(true, count); else stash(false, count);
            if (base + TOK < last) fetch(base + TOK, min(TOK, last - base - TOK));
        } else {
            for (int item = threadIdx.x; item < count * DPAD; item += THREADS) {
                const int t = item / DPAD, row = item % DPAD;
                float q = 0.f, k = 0.f;
                if (row < D) {
                    const T* src = projected + (size_t)(base + t) * a.ld;
                    if (MODE != 1) q = silu(to_float<T>(src[q_at + row])) * qfac[t];
                    k = silu(to_float<T>(src[k_at + row])) * kfac[t];
                }
                sq[t][row] = q;
                sk[t][row] = k;
            }
            for (int item = threadIdx.x; item < count * COLS; item += THREADS) {
                const int t = item / COLS, c = item % COLS;
                const int column = blockIdx.x * COLS + c;
                sv[t][c] = column < V
                    ? silu(to_float<T>(projected[(size_t)(base + t) * a.ld + v_at + column])) : 0.f;
            }
        }
        __syncthreads();
        // every lane of a warp reads the same k and q (a broadcast); the warp's share of a
        // token's output waits in shared memory for the other warps'
        if (scaled) {
            // S is kept divided by decay^(tokens of this group so far), k and q were staged times
            // decay^-(i+1) and decay^(i+1): an update and a sum are one multiply-add each
            for (int t = 0; t < count; ++t) {
                const float v = sv[t][col];
                float sum[4] = {0.f, 0.f, 0.f, 0.f};      // four chains of additions, not one
#pragma unroll
                for (int m = 0; m < DR / 4; ++m) {
                    const int at = 4 * (part + LANES * m);
                    const float4 k4 = *reinterpret_cast<const float4*>(&sk[t][at]);
                    const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
                    if (MODE == 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) S[4 * m + e] = fmaf(kk[e], v, S[4 * m + e]);
                    } else {
                        const float4 q4 = *reinterpret_cast<const float4*>(&sq[t][at]);
                        const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            S[4 * m + e] = fmaf(kk[e], v, S[4 * m + e]);
                            sum[e] = fmaf(S[4 * m + e], qq[e], sum[e]);
                        }
                    }
                }
                if (MODE != 1) parts[part][t][col] = (sum[0] + sum[1]) + (sum[2] + sum[3]);
            }
            const float back = qfac[count - 1];            // decay^count
#pragma unroll
            for (int i = 0; i < DR; ++i) S[i] *= back;
        } else {
            for (int t = 0; t < count; ++t) {
                const float v = sv[t][col];
                float sum = 0.f;
#pragma unroll
                for (int m = 0; m < DR / 4; ++m) {
                    const int at = 4 * (part + LANES * m);
                    const float4 k4 = *reinterpret_cast<const float4*>(&sk[t][at]);
                    const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
                    if (MODE == 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            S[4 * m + e] = fmaf(decay, S[4 * m + e], kk[e] * v);
                    } else {
                        const float4 q4 = *reinterpret_cast<const float4*>(&sq[t][at]);
                        const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            S[4 * m + e] = fmaf(decay, S[4 * m + e], kk[e] * v);
                            sum = fmaf(S[4 * m + e], qq[e], sum);
                        }
                    }
                }
                if (MODE != 1) parts[part][t][col] = sum;
            }
        }
        if (MODE != 1) {
            __syncthreads();
            // the four shares of every (token, column) are added in a fixed order
            for (int item = threadIdx.x; item < count * COLS; item += THREADS) {
                const int t = item / COLS, c = item % COLS;
                const int column = blockIdx.x * COLS + c;
                if (column < V)
                    a.o[(size_t)(base + t) * H * V + head * V + column] =
                        (parts[0][t][c] + parts[1][t][c]) + (parts[2][t][c] + parts[3][t][c]);
            }
        }
    }
    float* to = nullptr;
    if (MODE == 1) to = carried;
    else if (last_piece && a.write) to = slot;
    if (to != nullptr && live) {
#pragma unroll
        for (int m = 0; m < DR / 4; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = 4 * (part + LANES * m) + e;
                if (row < D) to[(size_t)row * V + j] = S[4 * m + e];
            }
    }
}

// carried[r][s] (what segment s adds from zero) becomes the state that segment s + 1 starts
// from: in = decay^segment * (state before segment s) + added(s). Written in place one segment
// later: carried[r][s + 1] <- in(s + 1), walking s upwards with the running value in a register;
// carried[r][0] gets the slot's state.
__global__ void lightning_chain_kernel(float* __restrict__ carried, const float* __restrict__ state,
                                       const int* __restrict__ slots,
                                       const int* __restrict__ request_start,
                                       const float* __restrict__ decay, int heads, long long per_head,
                                       int segment, int max_segments) {
    griddep_launch();
    griddep_wait();
    const int request = blockIdx.z, head = blockIdx.y;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per_head) return;
    const int count = request_start[request + 1] - request_start[request];
    const int pieces = (count + segment - 1) / segment;
    if (pieces <= 1) return;
    double exact = 1.0;                     // decay^segment, rounded once
    for (int s = 0; s < segment; ++s) exact *= (double)decay[head];
    const float power = (float)exact;
    float running = state[((size_t)slots[request] * heads + head) * per_head + i];
    float* at = carried + (((size_t)request * max_segments) * heads + head) * per_head + i;
    const size_t step = (size_t)heads * per_head;
    float added = at[0];
    at[0] = running;
    for (int s = 1; s < pieces; ++s) {
        running = fmaf(power, running, added);
        added = at[(size_t)s * step];        // what segment s adds (unused for the last one)
        at[(size_t)s * step] = running;      // what segment s starts from
    }
}

// out[t, c] = o[t, c] * rsqrt(mean_c(o[t, :]^2) + eps) * weight[c] * sigmoid(gate[t, c]).
template <typename T>
__global__ void lightning_finish_kernel(const float* __restrict__ o, const T* __restrict__ projected,
                                        int ld, int gate_at, const float* __restrict__ weight,
                                        T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const float* row = o + (size_t)t * width;
    float sum = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) sum = fmaf(row[c], row[c], sum);
    const float total = block_sum(sum, scratch);
    const float inv = rsqrtf(total / (float)width + eps);
    const T* gate = projected + (size_t)t * ld + gate_at;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float g = to_float<T>(gate[c]);
        out[(size_t)t * width + c] = from_float<T>(row[c] * inv * weight[c] / (1.f + expf(-g)));
    }
}

template <typename T, int DR>
cudaError_t launch_scan(const ScanArgs& a, int requests, int max_portion, cudaStream_t stream) {
    const int tiles = (a.value_dim + COLS - 1) / COLS;
    if (a.segment <= 0) {
        return launch_kernel(lightning_scan_kernel<T, DR, 0>, dim3(tiles, a.heads, requests),
                             dim3(THREADS), 0, stream, true, a);
    }
    const dim3 grid(tiles, a.heads, requests * a.max_segments);
    cudaError_t err = launch_kernel(lightning_scan_kernel<T, DR, 1>, grid, dim3(THREADS), 0, stream,
                                    true, a);
    if (err != cudaSuccess) return err;
    const long long per_head = (long long)a.key_dim * a.value_dim;
    err = launch_kernel(lightning_chain_kernel, dim3(ceil_div_host(per_head, 256), a.heads, requests),
                        dim3(256), 0, stream, true, a.carried, (const float*)a.state, a.slots,
                        a.request_start, a.decay, a.heads, per_head, a.segment, a.max_segments);
    if (err != cudaSuccess) return err;
    return launch_kernel(lightning_scan_kernel<T, DR, 2>, grid, dim3(THREADS), 0, stream, true, a);
}

template <typename T>
cudaError_t launch_scan_for(const ScanArgs& a, int requests, int max_portion, cudaStream_t stream) {
    const int d = a.key_dim;
    if (d <= 32) return launch_scan<T, 8>(a, requests, max_portion, stream);
    if (d <= 64) return launch_scan<T, 16>(a, requests, max_portion, stream);
    if (d <= 96) return launch_scan<T, 24>(a, requests, max_portion, stream);
    if (d <= 128) return launch_scan<T, 32>(a, requests, max_portion, stream);
    return launch_scan<T, 64>(a, requests, max_portion, stream);
}

}  // namespace

// Tokens per segment and segments per request for a step whose longest portion has
// `max_portion` tokens (0 segments: one run per request).
MLXONE_API int mlxone_lightning_segments(int max_portion, int* segment) {
    constexpr int SEGMENT = 64;
    *segment = 0;
    if (max_portion < 2 * SEGMENT) return 0;
    *segment = SEGMENT;
    return (max_portion + SEGMENT - 1) / SEGMENT;
}

// Floats of scratch: the 32-bit outputs [tokens, heads * V] and, for segmented steps, the
// carried states [requests, segments, heads, D, V].
MLXONE_API long long mlxone_lightning_scratch(int tokens, int requests, int max_portion, int heads,
                                              int key_dim, int value_dim) {
    int segment = 0;
    const int segments = mlxone_lightning_segments(max_portion, &segment);
    return (long long)tokens * heads * value_dim +
           (long long)requests * segments * heads * key_dim * value_dim;
}

MLXONE_API int mlxone_lightning(const void* projected, int ld, const float* decay,
                                const float* norm_weight, float eps, float* state, const int* slots,
                                const int* request_start, float* scratch, void* out, int tokens,
                                int requests, int max_portion, int heads, int key_dim, int value_dim,
                                int write, int dtype, cudaStream_t stream) {
    if (tokens == 0 || requests == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && requests > 0 && heads > 0 && key_dim > 0 && value_dim > 0,
                   "lightning: bad sizes");
    MLXONE_REQUIRE(key_dim <= 256, "lightning: key size %d exceeds 256", key_dim);
    MLXONE_REQUIRE(heads <= 65535 && requests <= 65535, "lightning: too many heads or requests");
    MLXONE_REQUIRE(ld >= 2 * heads * (key_dim + value_dim), "lightning: rows are too short");
    ScanArgs a;
    a.projected = projected; a.ld = ld; a.decay = decay; a.state = state; a.slots = slots;
    a.request_start = request_start; a.o = scratch; a.heads = heads; a.key_dim = key_dim;
    a.value_dim = value_dim; a.write = write;
    a.max_segments = mlxone_lightning_segments(max_portion, &a.segment);
    a.carried = scratch + (size_t)tokens * heads * value_dim;
    MLXONE_REQUIRE((long long)requests * (a.max_segments > 0 ? a.max_segments : 1) <= 65535,
                   "lightning: too many segments in one step");
    const int width = heads * value_dim;
    const int gate_at = 2 * heads * key_dim + width;
    const int threads = width >= 1024 ? 256 : 128;
    cudaError_t err;
    if (dtype == MLXONE_BF16) {
        err = launch_scan_for<__nv_bfloat16>(a, requests, max_portion, stream);
        if (err == cudaSuccess)
            err = launch_kernel(lightning_finish_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0,
                                stream, true, (const float*)scratch, (const __nv_bfloat16*)projected,
                                ld, gate_at, norm_weight, (__nv_bfloat16*)out, width, eps);
    } else {
        err = launch_scan_for<float>(a, requests, max_portion, stream);
        if (err == cudaSuccess)
            err = launch_kernel(lightning_finish_kernel<float>, dim3(tokens), dim3(threads), 0, stream,
                                true, (const float*)scratch, (const float*)projected, ld, gate_at,
                                norm_weight, (float*)out, width, eps);
    }
    if (err != cudaSuccess) {
        mlxone_set_error("lightning: launch failed: %s", cudaGetErrorString(err));
        return 2;
    }
    return 0;
}
