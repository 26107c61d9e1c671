// Mixers that carry a state of fixed size per request instead of a cache that grows: the plain kernels.
//
// Every kernel here finds a sequence's tokens through q_start[s] .. q_start[s + 1] and its state through
// state_slots[s], both on the device, so a step of single tokens launches the same grid whatever the slots hold and can
// be replayed from a captured graph.  A sequence's tokens are walked in order; the state is read once, kept in registers
// and written once.  State, decays, step sizes, gates of the recurrence and every sum are float;
// the projections come in the run dtype.
//
//   * li_causal_conv_silu / li_conv_state_shift: a depthwise causal convolution over the last `taps` inputs of each
//     channel followed by x / (1 + exp(-x)); the taps - 1 inputs before a portion come from the state, which the
//     second kernel then moves on (two launches: every token of the step reads the old state).
//   * li_ssm_scan: per head a state S [N, P]:  S = exp(-exp(A_log) dt) S + dt B x^T,  y = S^T C + D x, with
//     dt = softplus(dt_raw + dt_bias) per token and head, B and C shared by the heads of a group.
//   * li_decay_scan: per head a state S [d, dv]:  S = decay S + k v^T,  o = S^T q, with q, k, v passed through
//     x / (1 + exp(-x)) on the way in.
//   * li_gated_rmsnorm: RMSNorm in equal groups of a float row, with a gate before the norm (y * silu(z)) or after
//     it (norm(y) * sigmoid(g)).
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

constexpr int kMaxTaps = 8;

// in: [T, in_stride] with the C channels at column in_off; w [C, taps] (the last tap is the current token's), b [C];
// state [slots, state_stride] with the last taps - 1 inputs at state_off, oldest first, [taps - 1, C].
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, int in_stride, int in_off, const float* __restrict__ w, const float* __restrict__ b,
                                        const float* __restrict__ state, long long state_stride, long long state_off, const int* __restrict__ q_start,
                                        const int* __restrict__ seq_of_token, const int* __restrict__ slots, T* __restrict__ out, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = seq_of_token[t];
    const int q0 = q_start[s];
    const int li = t - q0;
    const float* st = state + (size_t)slots[s] * state_stride + state_off;
    float acc = b[c];
    for (int k = 0; k < taps; ++k) {
        const int i = li - (taps - 1) + k;
        const float v = i >= 0 ? to_float(in[(size_t)(q0 + i) * in_stride + in_off + c]) : st[(size_t)(taps - 1 + i) * C + c];
        acc = fmaf(w[(size_t)c * taps + k], v, acc);
    }
    out[(size_t)t * C + c] = from_float<T>(silu_f(acc));
}

template <typename T>
__global__ void conv_state_shift_kernel(const T* __restrict__ in, int in_stride, int in_off, float* __restrict__ state, long long state_stride,
                                        long long state_off, const int* __restrict__ q_start, const int* __restrict__ slots, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int q0 = q_start[s], n = q_start[s + 1] - q0;
    if (n <= 0) return;
    float* st = state + (size_t)slots[s] * state_stride + state_off;
    float keep[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
        if (j < taps - 1) {
            const int i = n - (taps - 1) + j;                    // index among the portion's inputs; negative: an older one
            keep[j] = i >= 0 ? to_float(in[(size_t)(q0 + i) * in_stride + in_off + c]) : st[(size_t)(taps - 1 + i) * C + c];
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j)
        if (j < taps - 1) st[(size_t)j * C + c] = keep[j];
}

// The two recurrences walk a sequence's tokens in order, but every column of a head's state moves on by itself:
// S[:, c] <- a_t S[:, c] + w_t[:] u_t[c],  out_t[c] = sum_i S[i, c] r_t[i].  So a column is the unit of work: eight lanes
// hold it in registers (element i with lane i % 8), four columns share a warp, four warps a block; a block stages the
// vectors of kStage tokens that all its columns need (w, r, and the scalars) in shared memory once, with the
// activations applied, and the columns then run through them with three shuffles a token for the sum.  The state is
// stored column by column ([head][column][element]) so that it is read and written in whole lines.
//
// Long portions are cut into chunks that run side by side (a sequence alone has too few columns to fill the GPU, and a
// walk over thousands of tokens is bound by its latency): `seg` names the chunks (begin, end, chunk, slot) and `mode` says
// which of three passes this is.  kScanLocal: every chunk from a state of zeros, no outputs, its end state to
// chunk_state[chunk].  li_scan_carry then walks each sequence's chunks in order, S <- decay(chunk) S + end state, and
// leaves in chunk_state[chunk] the state the chunk starts from (and the sequence's last state in its slot).  kScanApply:
// every chunk again from that state, with outputs.  Without `seg` (kScanWhole) a sequence is one piece, read from and
// written to its slot: steps of single tokens and short portions.
enum { kScanWhole = 0, kScanLocal = 1, kScanApply = 2 };
constexpr int kStage = 16;          // tokens staged at a time
constexpr int kColWarps = 4;        // warps a block
constexpr int kCols = kColWarps * 4;

__device__ __forceinline__ float oct_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v + __shfl_xor_sync(0xffffffffu, v, 4);
}

// xbc [T, C]: x (heads * P) | B (groups * N) | C (groups * N), after convolution and activation.  R = ceil(N / 8).
template <typename T, int R>
__global__ void __launch_bounds__(kColWarps * 32)
ssm_scan_kernel(const T* __restrict__ xbc, int C, const T* __restrict__ dt_raw, int dt_stride, const float* __restrict__ dt_bias,
                const float* __restrict__ A_log, const float* __restrict__ D, float* __restrict__ state, long long state_stride,
                const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ y, int heads, int P, int N, int groups,
                const int* __restrict__ seg, int mode, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    extern __shared__ float smem[];
    float* Bs = smem;                           // [kStage][N]
    float* Cs = Bs + (size_t)kStage * N;        // [kStage][N]
    float* xs = Cs + (size_t)kStage * N;        // [kStage][kCols]
    float* dts = xs + kStage * kCols;           // [kStage] step size
    float* das = dts + kStage;                  // [kStage] decay
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    int q0, q1, slot, chunk = 0;
    if (seg) {
        const int4 sg = reinterpret_cast<const int4*>(seg)[blockIdx.z];
        q0 = sg.x; q1 = sg.y; chunk = sg.z; slot = sg.w;
    } else {
        q0 = q_start[blockIdx.z]; q1 = q_start[blockIdx.z + 1]; slot = slots[blockIdx.z];
    }
    if (q1 <= q0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = lane & 7;
    const int col0 = blockIdx.x * kCols;
    const int c = col0 + warp * 4 + (lane >> 3);          // this lane's column of the head
    const bool live = c < P;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const size_t col_at = ((size_t)h * P + (live ? c : 0)) * N;
    float* st = state + (size_t)slot * state_stride + col_at;
    float* cst = chunk_state ? chunk_state + (size_t)chunk * heads * P * N + col_at : nullptr;
    const float* from = mode == kScanWhole ? st : cst;
    float S[R];
#pragma unroll
    for (int k = 0; k < R; ++k) S[k] = (mode != kScanLocal && live && m + 8 * k < N) ? from[m + 8 * k] : 0.0f;
    const float rate = expf(A_log[h]), bias = dt_bias[h], skip = D[h];
    if (mode == kScanLocal && blockIdx.x == 0 && warp == 0) {
        // the chunk's decay as a whole, for the pass that carries states from chunk to chunk
        float sum = 0.0f;
        for (int t = q0 + lane; t < q1; t += 32) sum += -rate * softplus_f(to_float(dt_raw[(size_t)t * dt_stride + h]) + bias);
        sum = warp_sum(sum);
        if (lane == 0) chunk_decay[(size_t)chunk * heads + h] = expf(sum);
    }
    for (int t0 = q0; t0 < q1; t0 += kStage) {
        const int nt = min(kStage, q1 - t0);
        __syncthreads();                                   // the stage before has been used up
        for (int tk = warp; tk < nt; tk += kColWarps) {
            const T* row = xbc + (size_t)(t0 + tk) * C;
            for (int n = lane; n < N; n += 32) {
                Bs[tk * N + n] = to_float(row[inner + g * N + n]);
                Cs[tk * N + n] = to_float(row[inner + (groups + g) * N + n]);
            }
        }
        for (int e = threadIdx.x; e < nt * kCols; e += blockDim.x) {
            const int tk = e / kCols, j = e - tk * kCols;
            xs[e] = col0 + j < P ? to_float(xbc[(size_t)(t0 + tk) * C + h * P + col0 + j]) : 0.0f;
        }
        if (threadIdx.x < nt) {
            const float dt = softplus_f(to_float(dt_raw[(size_t)(t0 + threadIdx.x) * dt_stride + h]) + bias);
            dts[threadIdx.x] = dt;
            das[threadIdx.x] = expf(-rate * dt);
        }
        __syncthreads();
#pragma unroll 4
        for (int tk = 0; tk < nt; ++tk) {
            const float x = xs[tk * kCols + warp * 4 + (lane >> 3)];
            const float dx = dts[tk] * x, decay = das[tk];
            const float* b = Bs + tk * N;
            const float* cc = Cs + tk * N;
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const int n = m + 8 * k;
                if (n < N) {
                    S[k] = fmaf(decay, S[k], b[n] * dx);
                    acc = fmaf(S[k], cc[n], acc);
                }
            }
            acc = oct_sum(acc);
            if (mode != kScanLocal && live && m == 0) y[(size_t)(t0 + tk) * inner + h * P + c] = fmaf(skip, x, acc);
        }
    }
    if (live && mode != kScanApply) {
        float* to = mode == kScanWhole ? st : cst;
#pragma unroll
        for (int k = 0; k < R; ++k)
            if (m + 8 * k < N) to[m + 8 * k] = S[k];
    }
}

// q, k [T, stride] at columns q_off + h d, k_off + h d; v at v_off + h dv; all before their activation.  R = ceil(d / 8).
template <typename T, int R>
__global__ void __launch_bounds__(kColWarps * 32)
decay_scan_kernel(const T* __restrict__ qkv, int stride, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                  float* __restrict__ out, int heads, int d, int dv, const int* __restrict__ seg, int mode, float* __restrict__ chunk_state) {
    extern __shared__ float smem[];
    float* qs = smem;                           // [kStage][d]
    float* ks = qs + (size_t)kStage * d;        // [kStage][d]
    float* vs = ks + (size_t)kStage * d;        // [kStage][kCols]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y;
    int q0, q1, slot, chunk = 0;
    if (seg) {
        const int4 sg = reinterpret_cast<const int4*>(seg)[blockIdx.z];
        q0 = sg.x; q1 = sg.y; chunk = sg.z; slot = sg.w;
    } else {
        q0 = q_start[blockIdx.z]; q1 = q_start[blockIdx.z + 1]; slot = slots[blockIdx.z];
    }
    if (q1 <= q0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = lane & 7;
    const int col0 = blockIdx.x * kCols;
    const int c = col0 + warp * 4 + (lane >> 3);
    const bool live = c < dv;
    const size_t col_at = ((size_t)h * dv + (live ? c : 0)) * d;
    float* st = state + (size_t)slot * state_stride + col_at;
    float* cst = chunk_state ? chunk_state + (size_t)chunk * heads * dv * d + col_at : nullptr;
    const float* from = mode == kScanWhole ? st : cst;
    float S[R];
#pragma unroll
    for (int k = 0; k < R; ++k) S[k] = (mode != kScanLocal && live && m + 8 * k < d) ? from[m + 8 * k] : 0.0f;
    const float lam = decay[h];
    for (int t0 = q0; t0 < q1; t0 += kStage) {
        const int nt = min(kStage, q1 - t0);
        __syncthreads();
        for (int tk = warp; tk < nt; tk += kColWarps) {
            const T* row = qkv + (size_t)(t0 + tk) * stride;
            for (int i = lane; i < d; i += 32) {
                if (mode != kScanLocal) qs[tk * d + i] = silu_f(to_float(row[q_off + h * d + i]));
                ks[tk * d + i] = silu_f(to_float(row[k_off + h * d + i]));
            }
        }
        for (int e = threadIdx.x; e < nt * kCols; e += blockDim.x) {
            const int tk = e / kCols, j = e - tk * kCols;
            vs[e] = col0 + j < dv ? silu_f(to_float(qkv[(size_t)(t0 + tk) * stride + v_off + h * dv + col0 + j])) : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int tk = 0; tk < nt; ++tk) {
            const float v = vs[tk * kCols + warp * 4 + (lane >> 3)];
            const float* kk = ks + tk * d;
            const float* qq = qs + tk * d;
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < R; ++k) {
                const int i = m + 8 * k;
                if (i < d) {
                    S[k] = fmaf(lam, S[k], kk[i] * v);
                    acc = fmaf(S[k], qq[i], acc);
                }
            }
            if (mode != kScanLocal) {
                acc = oct_sum(acc);
                if (live && m == 0) out[(size_t)(t0 + tk) * heads * dv + h * dv + c] = acc;
            }
        }
    }
    if (live && mode != kScanApply) {
        float* to = mode == kScanWhole ? st : cst;
#pragma unroll
        for (int k = 0; k < R; ++k)
            if (m + 8 * k < d) to[m + 8 * k] = S[k];
    }
}

// Between the two passes over chunks: for each run of chunks (a sequence's, in order) S starts as the slot's state;
// chunk_state[chunk] (the chunk's end state from zeros) is replaced by the state the chunk starts from, and
// S <- decay[chunk, head] S + end state.  The last S goes back to the slot.
__global__ void scan_carry_kernel(float* __restrict__ state, long long state_stride, float* __restrict__ chunk_state,
                                  const float* __restrict__ chunk_decay, const float* __restrict__ token_decay, const int* __restrict__ seg,
                                  const int* __restrict__ runs, int heads, int per_head) {
    pdl_launch_dependents();
    pdl_wait();
    const int first = runs[3 * blockIdx.y], count = runs[3 * blockIdx.y + 1], slot = runs[3 * blockIdx.y + 2];
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int elements = heads * per_head;
    if (e >= elements) return;
    const int h = e / per_head;
    float* st = state + (size_t)slot * state_stride + e;
    float S = *st;
    for (int c = first; c < first + count; ++c) {
        float* z = chunk_state + (size_t)c * elements + e;
        const float end_state = *z;
        *z = S;
        // the chunk's decay: given, or a constant per token and head to the power of the chunk's length
        const float dec = chunk_decay ? chunk_decay[(size_t)c * heads + h] : powf(token_decay[h], (float)(seg[4 * c + 1] - seg[4 * c]));
        S = fmaf(dec, S, end_state);
    }
    *st = S;
}

// One block per (token, group).  mode 0: v = y silu(z), out = v rinv w; mode 1: out = y rinv w sigmoid(z).
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int gate_stride, int gate_off, const float* __restrict__ w,
                                     float eps, int mode, T* __restrict__ out, int n, int groups) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x / groups, g = blockIdx.x - t * groups;
    const int gs = n / groups;
    const float* yr = y + (size_t)t * n + (size_t)g * gs;
    const T* zr = gate + (size_t)t * gate_stride + gate_off + (size_t)g * gs;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < gs; j += blockDim.x) {
        float v = yr[j];
        if (mode == 0) v *= silu_f(to_float(zr[j]));
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)gs + eps);
    T* o = out + (size_t)t * n + (size_t)g * gs;
    for (int j = threadIdx.x; j < gs; j += blockDim.x) {
        float v = yr[j];
        const float z = to_float(zr[j]);
        if (mode == 0) v = (v * silu_f(z)) * rinv * w[g * gs + j];
        else v = (v * rinv * w[g * gs + j]) * sigmoid_f(z);
        o[j] = from_float<T>(v);
    }
}

}  // namespace

LI_EXPORT int li_causal_conv_silu(const void* in, int dtype, int in_stride, int in_off, const float* w, const float* b, const float* state,
                                  long long state_stride, long long state_off, const int* q_start, const int* seq_of_token, const int* slots,
                                  void* out, int T, int C, int taps, cudaStream_t stream) {
    LI_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal convolution: %d taps (1..%d)", taps, kMaxTaps);
    LI_REQUIRE(C > 0 && in_off >= 0 && in_off + C <= in_stride, "causal convolution: %d channels at column %d of %d", C, in_off, in_stride);
    if (T == 0) return 0;
    LI_REQUIRE(T <= 65535, "causal convolution: %d tokens in one launch", T);
    const dim3 grid(ceil_div(C, 128), T);
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(causal_conv_silu_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, in_stride, in_off, w, b, state, state_stride,
                          state_off, q_start, seq_of_token, slots, (float*)out, C, taps);
    else if (dtype == LI_BF16)
        e = li_launch_pdl(causal_conv_silu_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, in_stride, in_off, w, b, state, state_stride,
                          state_off, q_start, seq_of_token, slots, (bf16*)out, C, taps);
    else
        return li_fail("causal convolution: unknown dtype %d", dtype);
    if (e != cudaSuccess) return li_fail("causal convolution: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("causal_conv_silu");
}

LI_EXPORT int li_conv_state_shift(const void* in, int dtype, int in_stride, int in_off, float* state, long long state_stride, long long state_off,
                                  const int* q_start, const int* slots, int S, int C, int taps, cudaStream_t stream) {
    LI_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal convolution: %d taps (1..%d)", taps, kMaxTaps);
    if (S == 0 || taps == 1) return 0;
    LI_REQUIRE(S <= 65535, "causal convolution: %d sequences in one launch", S);
    const dim3 grid(ceil_div(C, 128), S);
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(conv_state_shift_kernel<float>, grid, dim3(128), 0, stream, (const float*)in, in_stride, in_off, state, state_stride, state_off,
                          q_start, slots, C, taps);
    else if (dtype == LI_BF16)
        e = li_launch_pdl(conv_state_shift_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)in, in_stride, in_off, state, state_stride, state_off,
                          q_start, slots, C, taps);
    else
        return li_fail("causal convolution: unknown dtype %d", dtype);
    if (e != cudaSuccess) return li_fail("conv_state_shift: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("conv_state_shift");
}

template <typename T, int R>
static int launch_ssm(const void* xbc, int C, const void* dt_raw, int dt_stride, const float* dt_bias, const float* A_log, const float* D,
                      float* state, long long state_stride, const int* q_start, const int* slots, float* y, int S, int heads, int P, int N,
                      int groups, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    const size_t smem = ((size_t)2 * kStage * N + kStage * kCols + 2 * kStage) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(ssm_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = li_launch_pdl(ssm_scan_kernel<T, R>, dim3(ceil_div(P, kCols), heads, S), dim3(kColWarps * 32), smem, stream, (const T*)xbc, C,
                                  (const T*)dt_raw, dt_stride, dt_bias, A_log, D, state, state_stride, q_start, slots, y, heads, P, N, groups, seg, mode,
                                  chunk_state, chunk_decay);
    if (e != cudaSuccess) return li_fail("ssm_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("ssm_scan");
}

// The state of a slot: [heads][P][N] (a column of the head's N x P matrix at a time).
LI_EXPORT int li_ssm_scan(const void* xbc, int dtype, int C, const void* dt_raw, int dt_stride, const float* dt_bias, const float* A_log,
                          const float* D, float* state, long long state_stride, const int* q_start, const int* slots, float* y, int S, int heads,
                          int P, int N, int groups, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream) {
    LI_REQUIRE(mode == kScanWhole ? seg == nullptr : (seg != nullptr && chunk_state != nullptr && chunk_decay != nullptr && (uintptr_t)seg % 16 == 0),
               "state-space scan: pass %d needs the chunks, their states and their decays (or none of them)", mode);
    LI_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0, "state-space scan: %d heads in %d groups", heads, groups);
    LI_REQUIRE(P > 0 && N > 0 && N <= 256, "state-space scan: head size %d, state size %d (at most 256)", P, N);
    LI_REQUIRE(C == heads * P + 2 * groups * N, "state-space scan: %d channels for %d heads of %d and %d groups of %d", C, heads, P, groups, N);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "state-space scan: unknown dtype %d", dtype);
    if (S == 0) return 0;
    LI_REQUIRE(S <= 65535 && heads <= 65535, "state-space scan: %d sequences or %d heads in one launch", S, heads);
#define LI_SCAN(RR)                                                                                                                            \
    return dtype == LI_F32 ? launch_ssm<float, RR>(xbc, C, dt_raw, dt_stride, dt_bias, A_log, D, state, state_stride, q_start, slots, y, S, heads, \
                                                   P, N, groups, seg, mode, chunk_state, chunk_decay, stream)                                  \
                           : launch_ssm<bf16, RR>(xbc, C, dt_raw, dt_stride, dt_bias, A_log, D, state, state_stride, q_start, slots, y, S, heads,  \
                                                  P, N, groups, seg, mode, chunk_state, chunk_decay, stream)
    if (N <= 16) { LI_SCAN(2); }
    if (N <= 32) { LI_SCAN(4); }
    if (N <= 64) { LI_SCAN(8); }
    if (N <= 128) { LI_SCAN(16); }
    LI_SCAN(32);
#undef LI_SCAN
}

template <typename T, int R>
static int launch_decay(const void* qkv, int stride, int q_off, int k_off, int v_off, const float* decay, float* state, long long state_stride,
                        const int* q_start, const int* slots, float* out, int S, int heads, int d, int dv, const int* seg, int mode,
                        float* chunk_state, cudaStream_t stream) {
    const size_t smem = ((size_t)2 * kStage * d + kStage * kCols) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = li_launch_pdl(decay_scan_kernel<T, R>, dim3(ceil_div(dv, kCols), heads, S), dim3(kColWarps * 32), smem, stream, (const T*)qkv, stride,
                                  q_off, k_off, v_off, decay, state, state_stride, q_start, slots, out, heads, d, dv, seg, mode, chunk_state);
    if (e != cudaSuccess) return li_fail("decay_scan: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("decay_scan");
}

// The state of a slot: [heads][dv][d] (a column of the head's d x dv matrix at a time).
LI_EXPORT int li_decay_scan(const void* qkv, int dtype, int stride, int q_off, int k_off, int v_off, const float* decay, float* state,
                            long long state_stride, const int* q_start, const int* slots, float* out, int S, int heads, int d, int dv,
                            const int* seg, int mode, float* chunk_state, cudaStream_t stream) {
    LI_REQUIRE(mode == kScanWhole ? seg == nullptr : (seg != nullptr && chunk_state != nullptr && (uintptr_t)seg % 16 == 0),
               "decay scan: pass %d needs the chunks and their states (or none of them)", mode);
    LI_REQUIRE(heads > 0 && d > 0 && d <= 256 && dv > 0, "decay scan: %d heads of %d x %d (keys of at most 256)", heads, d, dv);
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "decay scan: unknown dtype %d", dtype);
    if (S == 0) return 0;
    LI_REQUIRE(S <= 65535 && heads <= 65535, "decay scan: %d sequences or %d heads in one launch", S, heads);
#define LI_SCAN(RR)                                                                                                                          \
    return dtype == LI_F32 ? launch_decay<float, RR>(qkv, stride, q_off, k_off, v_off, decay, state, state_stride, q_start, slots, out, S, heads, \
                                                     d, dv, seg, mode, chunk_state, stream)                                                  \
                           : launch_decay<bf16, RR>(qkv, stride, q_off, k_off, v_off, decay, state, state_stride, q_start, slots, out, S, heads,  \
                                                    d, dv, seg, mode, chunk_state, stream)
    if (d <= 16) { LI_SCAN(2); }
    if (d <= 32) { LI_SCAN(4); }
    if (d <= 64) { LI_SCAN(8); }
    if (d <= 128) { LI_SCAN(16); }
    LI_SCAN(32);
#undef LI_SCAN
}

// See scan_carry_kernel.  runs: triples (first chunk, chunks, slot); per_head: state elements of one head.  The decay of a
// chunk and head: chunk_decay[chunk, head], or (chunk_decay null) token_decay[head] to the power of the chunk's length.
LI_EXPORT int li_scan_carry(float* state, long long state_stride, float* chunk_state, const float* chunk_decay, const float* token_decay,
                            const int* seg, const int* runs, int nruns, int heads, int per_head, cudaStream_t stream) {
    LI_REQUIRE(heads > 0 && per_head > 0, "scan carry: %d heads of %d elements", heads, per_head);
    LI_REQUIRE(chunk_decay != nullptr || (token_decay != nullptr && seg != nullptr), "scan carry: no decay given");
    if (nruns == 0) return 0;
    LI_REQUIRE(nruns <= 65535, "scan carry: %d sequences in one launch", nruns);
    cudaError_t e = li_launch_pdl(scan_carry_kernel, dim3(ceil_div(heads * per_head, 256), nruns), dim3(256), 0, stream, state, state_stride, chunk_state,
                                  chunk_decay, token_decay, seg, runs, heads, per_head);
    if (e != cudaSuccess) return li_fail("scan_carry: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("scan_carry");
}

LI_EXPORT int li_gated_rmsnorm(const float* y, const void* gate, int dtype, int gate_stride, int gate_off, const float* w, float eps, int mode,
                               void* out, int T, int n, int groups, cudaStream_t stream) {
    LI_REQUIRE(n > 0 && groups > 0 && n % groups == 0, "gated norm: %d columns in %d groups", n, groups);
    LI_REQUIRE(mode == 0 || mode == 1, "gated norm: unknown mode %d", mode);
    LI_REQUIRE(gate_off >= 0 && gate_off + n <= gate_stride, "gated norm: gate at column %d of %d for %d columns", gate_off, gate_stride, n);
    if (T == 0) return 0;
    const long long blocks = (long long)T * groups;
    LI_REQUIRE(blocks < (1LL << 31), "gated norm: too many rows");
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(gated_rmsnorm_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, y, (const float*)gate, gate_stride, gate_off, w, eps,
                          mode, (float*)out, n, groups);
    else if (dtype == LI_BF16)
        e = li_launch_pdl(gated_rmsnorm_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, y, (const bf16*)gate, gate_stride, gate_off, w, eps,
                          mode, (bf16*)out, n, groups);
    else
        return li_fail("gated norm: unknown dtype %d", dtype);
    if (e != cudaSuccess) return li_fail("gated_rmsnorm: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("gated_rmsnorm");
}
