// Hyper-connections: the residual stream as s parallel streams, xs [tokens, s, width] float.
//
// A sublayer reads u = sum_s in[s] xs[s], runs on norm(u), and its output y is written back as
//   xs'[r] = sum_s mix[s, r] xs[s] + out[r] y          (all streams at once, from the old ones).
// Two kernels, one block per token, everything in float:
//   * read:   u (with given read weights, or the plain sum of the streams) -> RMSNorm -> run dtype; rows may be gathered
//             (the final norm on the rows whose logits are wanted);
//   * update: the write-back of one sublayer and, in the same pass, the read and norm of the next one, so that the
//             streams cross memory once per sublayer as the single stream does in the add + norm kernel.
// The streams of an element are independent of every other element, so the update is in place.
// Also here: learned absolute positions added to the stream, and the copy of one stream into s.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxStreams = 8;

// four neighbouring elements at a time where the width allows (16-byte loads and stores of the streams)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<const unsigned*>(&a);
    r.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}
__device__ __forceinline__ float4 fma4(float a, float4 x, float4 acc) {
    return make_float4(fmaf(a, x.x, acc.x), fmaf(a, x.y, acc.y), fmaf(a, x.z, acc.z), fmaf(a, x.w, acc.w));
}

template <typename T>
__global__ void hc_read_norm_kernel(const float* __restrict__ xs, const float* __restrict__ in_w, const int* __restrict__ rows,
                                    const float* __restrict__ w, float eps, T* __restrict__ out, int rows_in, int s, int H) {
    extern __shared__ __align__(16) float u_row[];
    __shared__ float scratch[32];
    __shared__ float wi[kMaxStreams];
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x < s) wi[threadIdx.x] = in_w ? in_w[threadIdx.x] : 1.0f;
    __syncthreads();
    const int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    if (src < 0 || src >= rows_in) src = 0;
    const float* x = xs + (size_t)src * s * H;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float u = 0.0f;
#pragma unroll
        for (int a = 0; a < kMaxStreams; ++a)
            if (a < s) u = fmaf(wi[a], x[(size_t)a * H + j], u);
        u_row[j] = u;
        ss += u * u;
    }
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = from_float<T>((w[j] * u_row[j]) * rinv);
}

template <typename T>
__global__ void hc_update_kernel(float* __restrict__ xs, const T* __restrict__ y, const T* __restrict__ y2, float s1, float s2,
                                 const float* __restrict__ mix, const float* __restrict__ out_w,
                                 const float* __restrict__ next_in, const float* __restrict__ next_w, float eps, T* __restrict__ next_out,
                                 int s, int H) {
    extern __shared__ __align__(16) float u_row[];
    __shared__ float scratch[32];
    __shared__ float m[kMaxStreams * kMaxStreams], wo[kMaxStreams], wi[kMaxStreams];
    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < s * s; i += blockDim.x) m[i] = mix[i];
    if (threadIdx.x < s) {
        wo[threadIdx.x] = out_w[threadIdx.x];
        wi[threadIdx.x] = next_in ? next_in[threadIdx.x] : 0.0f;
    }
    __syncthreads();
    const int t = blockIdx.x;
    float* x = xs + (size_t)t * s * H;
    float ss = 0.0f;
    if ((H & 3) == 0) {
        for (int j = 4 * threadIdx.x; j < H; j += 4 * blockDim.x) {
            float4 old[kMaxStreams];
#pragma unroll
            for (int a = 0; a < kMaxStreams; ++a) old[a] = a < s ? load4(x + (size_t)a * H + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 yj = load4(y + (size_t)t * H + j);
            if (y2) {
                const float4 b = load4(y2 + (size_t)t * H + j);
                yj = make_float4(fmaf(s1, yj.x, s2 * b.x), fmaf(s1, yj.y, s2 * b.y), fmaf(s1, yj.z, s2 * b.z), fmaf(s1, yj.w, s2 * b.w));
            }
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < kMaxStreams; ++r) {
                if (r < s) {
                    float4 v = make_float4(wo[r] * yj.x, wo[r] * yj.y, wo[r] * yj.z, wo[r] * yj.w);
#pragma unroll
                    for (int a = 0; a < kMaxStreams; ++a)
                        if (a < s) v = fma4(m[a * s + r], old[a], v);
                    store4(x + (size_t)r * H + j, v);
                    u = fma4(wi[r], v, u);
                }
            }
            if (next_out) {
                store4(u_row + j, u);
                ss += u.x * u.x;
                ss += u.y * u.y;
                ss += u.z * u.z;
                ss += u.w * u.w;
            }
        }
    } else {
        for (int j = threadIdx.x; j < H; j += blockDim.x) {
            float old[kMaxStreams];
#pragma unroll
            for (int a = 0; a < kMaxStreams; ++a) old[a] = a < s ? x[(size_t)a * H + j] : 0.0f;
            float yj = to_float(y[(size_t)t * H + j]);
            if (y2) yj = fmaf(s1, yj, s2 * to_float(y2[(size_t)t * H + j]));        // the sublayer's output as a weighted sum of two
            float u = 0.0f;
#pragma unroll
            for (int r = 0; r < kMaxStreams; ++r) {
                if (r < s) {
                    float v = wo[r] * yj;
#pragma unroll
                    for (int a = 0; a < kMaxStreams; ++a)
                        if (a < s) v = fmaf(m[a * s + r], old[a], v);
                    x[(size_t)r * H + j] = v;
                    u = fmaf(wi[r], v, u);
                }
            }
            if (next_out) {
                u_row[j] = u;
                ss += u * u;
            }
        }
    }
    if (!next_out) return;
    ss = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = next_out + (size_t)t * H;
    if ((H & 3) == 0) {
        for (int j = 4 * threadIdx.x; j < H; j += 4 * blockDim.x) {
            const float4 u = load4(u_row + j), w4 = load4(next_w + j);
            store4(o + j, make_float4((w4.x * u.x) * rinv, (w4.y * u.y) * rinv, (w4.z * u.z) * rinv, (w4.w * u.w) * rinv));
        }
    } else {
        for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = from_float<T>((next_w[j] * u_row[j]) * rinv);
    }
}

__global__ void hc_expand_kernel(const float* __restrict__ x, float* __restrict__ xs, int s, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float v = x[(size_t)t * H + j];
        for (int a = 0; a < s; ++a) xs[((size_t)t * s + a) * H + j] = v;
    }
}

template <typename T>
__global__ void add_position_rows_kernel(float* __restrict__ x, const T* __restrict__ table, const int* __restrict__ positions, int H, int P) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int p = positions[t];
    p = p < 0 ? 0 : (p >= P ? P - 1 : p);              // the host refuses positions beyond the table; never read outside it
    for (int j = threadIdx.x; j < H; j += blockDim.x) x[(size_t)t * H + j] += to_float(table[(size_t)p * H + j]);
}

}  // namespace

// out[r] = RMSNorm(sum_s in_w[s] xs[rows[r], s]) * w.  in_w null: the plain sum; rows null: every row in order.
LI_EXPORT int li_hc_read_norm(const float* xs, const float* in_w, const int* rows, const float* w, float eps, void* out, int dtype, int R,
                              int T, int s, int H, cudaStream_t stream) {
    LI_REQUIRE(s >= 1 && s <= kMaxStreams, "hyper-connections: %d streams (1..%d)", s, kMaxStreams);
    LI_REQUIRE(H > 0 && (size_t)H * 4 <= 200 * 1024, "hyper-connections: width %d", H);
    if (R == 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    cudaError_t e;
    if (dtype == LI_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hc_read_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = li_launch_pdl(hc_read_norm_kernel<float>, dim3(R), dim3(kThreads), smem, stream, xs, in_w, rows, w, eps, (float*)out, T, s, H);
    } else if (dtype == LI_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hc_read_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = li_launch_pdl(hc_read_norm_kernel<bf16>, dim3(R), dim3(kThreads), smem, stream, xs, in_w, rows, w, eps, (bf16*)out, T, s, H);
    } else {
        return li_fail("hyper-connections: unknown dtype %d", dtype);
    }
    if (e != cudaSuccess) return li_fail("hc_read_norm: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("hc_read_norm");
}

// xs[t, r] = sum_s mix[s, r] xs[t, s] + out_w[r] y[t]; then, unless next_out is null,
// next_out[t] = RMSNorm(sum_r next_in[r] xs[t, r]) * next_w.  With y2, the sublayer's output is s1 y + s2 y2 (two mixers
// side by side), summed in float.
LI_EXPORT int li_hc_update(float* xs, const void* y, const void* y2, float s1, float s2, int dtype, const float* mix, const float* out_w,
                           const float* next_in, const float* next_w, float eps, void* next_out, int T, int s, int H, cudaStream_t stream) {
    LI_REQUIRE(s >= 1 && s <= kMaxStreams, "hyper-connections: %d streams (1..%d)", s, kMaxStreams);
    LI_REQUIRE(H > 0 && (size_t)H * 4 <= 200 * 1024, "hyper-connections: width %d", H);
    LI_REQUIRE(next_out == nullptr || (next_in != nullptr && next_w != nullptr), "hc_update: the next read needs its weights");
    if (T == 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    cudaError_t e;
    if (dtype == LI_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hc_update_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = li_launch_pdl(hc_update_kernel<float>, dim3(T), dim3(kThreads), smem, stream, xs, (const float*)y, (const float*)y2, s1, s2, mix, out_w, next_in, next_w, eps,
                          (float*)next_out, s, H);
    } else if (dtype == LI_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(hc_update_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = li_launch_pdl(hc_update_kernel<bf16>, dim3(T), dim3(kThreads), smem, stream, xs, (const bf16*)y, (const bf16*)y2, s1, s2, mix, out_w, next_in, next_w, eps,
                          (bf16*)next_out, s, H);
    } else {
        return li_fail("hyper-connections: unknown dtype %d", dtype);
    }
    if (e != cudaSuccess) return li_fail("hc_update: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("hc_update");
}

// xs[t, a] = x[t] for a = 0 .. s-1.
LI_EXPORT int li_hc_expand(const float* x, float* xs, int T, int s, int H, cudaStream_t stream) {
    LI_REQUIRE(s >= 1 && H > 0, "hc_expand: %d streams of width %d", s, H);
    if (T == 0) return 0;
    cudaError_t e = li_launch_pdl(hc_expand_kernel, dim3(T), dim3(kThreads), 0, stream, x, xs, s, H);
    if (e != cudaSuccess) return li_fail("hc_expand: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("hc_expand");
}

// x[t] += table[positions[t]] (learned absolute positions; table [P, H] in the run dtype).
LI_EXPORT int li_add_position_rows(float* x, const void* table, int dtype, const int* positions, int T, int H, int P, cudaStream_t stream) {
    LI_REQUIRE(H > 0 && P > 0, "add_position_rows: table of %d rows of %d", P, H);
    if (T == 0) return 0;
    cudaError_t e;
    if (dtype == LI_F32) e = li_launch_pdl(add_position_rows_kernel<float>, dim3(T), dim3(kThreads), 0, stream, x, (const float*)table, positions, H, P);
    else if (dtype == LI_BF16) e = li_launch_pdl(add_position_rows_kernel<bf16>, dim3(T), dim3(kThreads), 0, stream, x, (const bf16*)table, positions, H, P);
    else return li_fail("add_position_rows: unknown dtype %d", dtype);
    if (e != cudaSuccess) return li_fail("add_position_rows: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("add_position_rows");
}
