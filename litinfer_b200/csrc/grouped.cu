// Products in groups, and the routing of a mixture of experts around them.
//
//   li_grouped_linear: G products out_g = a_g w_g^T with one matrix w_g [N, K] per group (w is [G, N, K]), two ways:
//     * rows in groups (row_offsets [G + 1] on the device): group g owns the rows row_offsets[g] .. row_offsets[g + 1] - 1 of
//       a [M, lda] and of out [M, ldc], all columns alike: the experts of a mixture, tokens sorted by expert;
//     * columns in groups (row_offsets NULL): every group takes all M rows, its inputs at column g * a_gcol of a and its
//       outputs at column g * c_gcol of out: a map per head.
//     float32 (and bfloat16 shapes the other kernel refuses): CUDA-core tiles of 64 x 64 x 16.  bfloat16 with K a
//     multiple of 8: mma.sync tiles of 64 x 64 x 32 (four warps of 16 rows, operands through shared memory with
//     16-byte asynchronous copies, two stages).  Either way float accumulation, each output summed over k in ascending
//     order by one thread: a row's result does not depend on which rows stand beside it.
//   li_moe_route:   scores = sigmoid(logits), the `top` largest per token (the lower index wins a tie); the scores of the
//     chosen are the weights as they are, not renormalised.
//   li_moe_sort:    a stable counting sort of the (token, choice) pairs by expert: offsets per expert, the pair at each
//     sorted place, and each pair's place.  One block per expert walks the pairs in order, so the result is the same
//     whatever runs beside it.
//   li_moe_gather:  sorted row r = weight(pair) * h[token(pair)] (the weight goes on the expert's input), or the plain row.
//   li_moe_combine: y[t] = sum over the token's choices of the sorted rows (times the weight, when it goes on the output),
//     summed in float in the order of the choices.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(256)
grouped_linear_kernel(const Tin* __restrict__ A, int lda, int a_gcol, const Tin* __restrict__ W, Tout* __restrict__ C, int ldc, int c_gcol,
                      const int* __restrict__ row_offsets, int M, int N, int K, int G) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    int g, m0, m_end;
    if (row_offsets) {
        // blockIdx.y counts row tiles over all groups: find the group this one falls into
        int tile = blockIdx.y;
        g = 0;
        while (g < G) {
            const int rows = row_offsets[g + 1] - row_offsets[g];
            const int tiles = (rows + BM - 1) / BM;
            if (tile < tiles) break;
            tile -= tiles;
            ++g;
        }
        if (g >= G) return;
        m0 = row_offsets[g] + tile * BM;
        m_end = row_offsets[g + 1];
    } else {
        g = blockIdx.z;
        m0 = blockIdx.y * BM;
        m_end = M;
    }
    const Tin* a = A + (size_t)g * a_gcol;
    const Tin* w = W + (size_t)g * N * K;
    Tout* c = C + (size_t)g * c_gcol;
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * BN;
    const int tx = tid & 15, ty = tid >> 4;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        float av[4], wv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int am = m0 + lr, wn = n0 + lr;
            av[q] = (am < m_end && k < K) ? to_float(a[(size_t)am * lda + k]) : 0.0f;
            wv[q] = (wn < N && k < K) ? to_float(w[(size_t)wn * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            As[lk + q][lr] = av[q];
            Ws[lk + q][lr] = wv[q];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float ar[TM], wr[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ar[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wr[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= m_end) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) c[(size_t)m * ldc + n] = from_float<Tout>(acc[i][j]);
        }
    }
}

// ---- the same on the tensor cores (bfloat16) ----------------------------------------------------------------------------

constexpr int MK = 32, MPAD = 8;          // k elements a stage; padding of a shared row (its 80 bytes keep 16-byte alignment)

__device__ __forceinline__ void cp16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;                               // 0: the destination is filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128)
grouped_mma_kernel(const bf16* __restrict__ A, int lda, int a_gcol, const bf16* __restrict__ W, bf16* __restrict__ C, int ldc, int c_gcol,
                   const int* __restrict__ row_offsets, int M, int N, int K, int G) {
    __shared__ __align__(16) bf16 As[2][BM][MK + MPAD];
    __shared__ __align__(16) bf16 Ws[2][BN][MK + MPAD];
    pdl_launch_dependents();
    pdl_wait();
    int g, m0, m_end;
    if (row_offsets) {
        int tile = blockIdx.y;
        g = 0;
        while (g < G) {
            const int rows = row_offsets[g + 1] - row_offsets[g];
            const int tiles = (rows + BM - 1) / BM;
            if (tile < tiles) break;
            tile -= tiles;
            ++g;
        }
        if (g >= G) return;
        m0 = row_offsets[g] + tile * BM;
        m_end = row_offsets[g + 1];
    } else {
        g = blockIdx.z;
        m0 = blockIdx.y * BM;
        m_end = M;
    }
    const bf16* a = A + (size_t)g * a_gcol;
    const bf16* w = W + (size_t)g * N * K;
    bf16* c = C + (size_t)g * c_gcol;
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gq = lane >> 2, t = lane & 3;
    auto load = [&](int stage, int k0) {
        // 64 rows of 4 chunks of 8 elements for each operand: 256 chunks each, two per thread
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * 128;
            const int r = idx >> 2, ch = idx & 3;
            const int k = k0 + ch * 8;
            const bool ka = k < K;
            const bool va = ka && m0 + r < m_end, vw = ka && n0 + r < N;
            cp16(&As[stage][r][ch * 8], va ? a + (size_t)(m0 + r) * lda + k : a, va);
            cp16(&Ws[stage][r][ch * 8], vw ? w + (size_t)(n0 + r) * K + k : w, vw);
        }
        asm volatile("cp.async.commit_group;");
    };
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    load(0, 0);
    int stage = 0;
    for (int k0 = 0; k0 < K; k0 += MK, stage ^= 1) {
        if (k0 + MK < K) {
            load(stage ^ 1, k0 + MK);
            asm volatile("cp.async.wait_group 1;");
        } else {
            asm volatile("cp.async.wait_group 0;");
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < MK; ks += 16) {
            const bf16* ar = &As[stage][warp * 16 + gq][ks + 2 * t];
            const unsigned a0 = *reinterpret_cast<const unsigned*>(ar), a1 = *reinterpret_cast<const unsigned*>(ar + 8 * (MK + MPAD));
            const unsigned a2 = *reinterpret_cast<const unsigned*>(ar + 8), a3 = *reinterpret_cast<const unsigned*>(ar + 8 * (MK + MPAD) + 8);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bf16* wr = &Ws[stage][j * 8 + gq][ks + 2 * t];
                mma16816(acc[j], a0, a1, a2, a3, *reinterpret_cast<const unsigned*>(wr), *reinterpret_cast<const unsigned*>(wr + 8));
            }
        }
        __syncthreads();                     // the stage is overwritten by the load the next iteration issues
    }
    const int r_lo = m0 + warp * 16 + gq, r_hi = r_lo + 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int n = n0 + j * 8 + 2 * t;
        if (n < N) {
            if (r_lo < m_end) c[(size_t)r_lo * ldc + n] = __float2bfloat16_rn(acc[j][0]);
            if (r_hi < m_end) c[(size_t)r_hi * ldc + n] = __float2bfloat16_rn(acc[j][2]);
        }
        if (n + 1 < N) {
            if (r_lo < m_end) c[(size_t)r_lo * ldc + n + 1] = __float2bfloat16_rn(acc[j][1]);
            if (r_hi < m_end) c[(size_t)r_hi * ldc + n + 1] = __float2bfloat16_rn(acc[j][3]);
        }
    }
}

// ---- routing ---------------------------------------------------------------------------------------------------------

constexpr int kMaxExpertsPerLane = 8;       // experts <= 256

__global__ void moe_route_kernel(const float* __restrict__ logits, int T, int E, int top, int* __restrict__ ids, float* __restrict__ weights) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    float s[kMaxExpertsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < E ? 1.0f / (1.0f + expf(-logits[(size_t)t * E + e])) : -1.0f;      // scores lie in (0, 1): -1 never wins
    }
    for (int k = 0; k < top; ++k) {
        float best = -2.0f;
        int arg = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            const int e = lane + 32 * i;
            if (s[i] > best) best = s[i], arg = e;                 // ascending e within a lane: the lower index keeps a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
        }
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            weights[(size_t)t * top + k] = best;
        }
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
            if (lane + 32 * i == arg) s[i] = -1.0f;
    }
}

// One block per expert.  n pairs (token, choice) in order; ids[i] is pair i's expert.
__global__ void moe_sort_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ offsets, int* __restrict__ pair_at,
                                int* __restrict__ place_of) {
    __shared__ int warp_total[32];
    __shared__ int less_total[32];
    __shared__ int base_eq;
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // how many pairs go to experts before this one: where this expert's rows start
    int less = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) less += ids[i] < e ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) less += __shfl_xor_sync(0xffffffffu, less, o);
    if (lane == 0) less_total[warp] = less;
    if (threadIdx.x == 0) base_eq = 0;
    __syncthreads();
    int start = 0;
    for (int w = 0; w < nwarps; ++w) start += less_total[w];
    // this expert's pairs, in order
    for (int base = 0; base < n; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const bool mine = i < n && ids[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_total[warp] = __popc(ballot);
        __syncthreads();
        int before = base_eq;
        for (int w = 0; w < warp; ++w) before += warp_total[w];
        if (mine) {
            const int place = start + before + __popc(ballot & ((1u << lane) - 1u));
            pair_at[place] = i;
            place_of[i] = place;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < nwarps; ++w) total += warp_total[w];
            base_eq += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        offsets[e] = start;
        if (e == E - 1) offsets[E] = start + base_eq;
    }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ pair_at, const float* __restrict__ weights, int top, int H,
                                  T* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int pair = pair_at[r];
    const T* src = h + (size_t)(pair / top) * H;
    T* dst = out + (size_t)r * H;
    if (weights) {
        const float w = weights[pair];
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = from_float<T>(w * to_float(src[i]));
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
    }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ place_of, const float* __restrict__ weights, int top, int H,
                                   T* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.0f;
        for (int k = 0; k < top; ++k) {
            const float v = to_float(rows[(size_t)place_of[(size_t)t * top + k] * H + i]);
            acc += weights ? weights[(size_t)t * top + k] * v : v;
        }
        y[(size_t)t * H + i] = from_float<T>(acc);
    }
}

}  // namespace

LI_EXPORT int li_grouped_linear(const void* a, int lda, int a_gcol, const void* w, void* out, int ldc, int c_gcol, const int* row_offsets, int dtype,
                                int M, int N, int K, int G, cudaStream_t stream) {
    LI_REQUIRE(M >= 0 && N > 0 && K > 0 && G > 0, "grouped_linear: bad sizes M=%d N=%d K=%d G=%d", M, N, K, G);
    LI_REQUIRE(lda >= K && ldc >= N, "grouped_linear: rows of %d and %d elements cannot hold K=%d and N=%d", lda, ldc, K, N);
    LI_REQUIRE(row_offsets == nullptr || (a_gcol == 0 && c_gcol == 0), "grouped_linear: groups are rows or columns, not both");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "grouped_linear: unknown dtype %d", dtype);
    if (M == 0) return 0;
    const int row_tiles = ceil_div(M, BM);
    const dim3 grid(ceil_div(N, BN), row_offsets ? row_tiles + G : row_tiles, row_offsets ? 1 : G);
    LI_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "grouped_linear: too many tiles for one launch");
    cudaError_t e;
    // 16-byte copies: every row and every group's first column on a 16-byte boundary
    const bool aligned = K % 8 == 0 && lda % 8 == 0 && a_gcol % 8 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0;
    if (dtype == LI_BF16 && aligned)
        e = li_launch_pdl(grouped_mma_kernel, grid, dim3(128), 0, stream, (const bf16*)a, lda, a_gcol, (const bf16*)w, (bf16*)out, ldc, c_gcol,
                          row_offsets, M, N, K, G);
    else if (dtype == LI_F32)
        e = li_launch_pdl(grouped_linear_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)a, lda, a_gcol, (const float*)w, (float*)out,
                          ldc, c_gcol, row_offsets, M, N, K, G);
    else
        e = li_launch_pdl(grouped_linear_kernel<bf16, bf16>, grid, dim3(256), 0, stream, (const bf16*)a, lda, a_gcol, (const bf16*)w, (bf16*)out, ldc,
                          c_gcol, row_offsets, M, N, K, G);
    if (e != cudaSuccess) return li_fail("grouped_linear: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("grouped_linear");
}

LI_EXPORT int li_moe_route(const float* logits, int T, int E, int top, int* ids, float* weights, cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && E > 0 && top > 0 && top <= E, "moe_route: %d of %d experts", top, E);
    LI_REQUIRE(E <= 32 * kMaxExpertsPerLane, "moe_route: %d experts are more than %d", E, 32 * kMaxExpertsPerLane);
    if (T == 0) return 0;
    const cudaError_t e = li_launch_pdl(moe_route_kernel, dim3(ceil_div(T, 4)), dim3(128), 0, stream, logits, T, E, top, ids, weights);
    if (e != cudaSuccess) return li_fail("moe_route: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_route");
}

LI_EXPORT int li_moe_sort(const int* ids, int n, int E, int* offsets, int* pair_at, int* place_of, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && E > 0, "moe_sort: bad sizes");
    const cudaError_t e = li_launch_pdl(moe_sort_kernel, dim3(E), dim3(256), 0, stream, ids, n, E, offsets, pair_at, place_of);
    if (e != cudaSuccess) return li_fail("moe_sort: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_sort");
}

// out [n, H]: row r is h[pair_at[r] / top], times weights[pair_at[r]] if weights is given.
LI_EXPORT int li_moe_gather(const void* h, int dtype, const int* pair_at, const float* weights, int n, int top, int H, void* out, cudaStream_t stream) {
    LI_REQUIRE(n >= 0 && top > 0 && H > 0, "moe_gather: bad sizes");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "moe_gather: unknown dtype %d", dtype);
    if (n == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(moe_gather_kernel<float>, dim3(n), dim3(threads), 0, stream, (const float*)h, pair_at, weights, top, H, (float*)out);
    else
        e = li_launch_pdl(moe_gather_kernel<bf16>, dim3(n), dim3(threads), 0, stream, (const bf16*)h, pair_at, weights, top, H, (bf16*)out);
    if (e != cudaSuccess) return li_fail("moe_gather: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_gather");
}

// y [T, H]: y[t] = sum_k rows[place_of[t * top + k]] (times weights[t * top + k] if weights is given).
LI_EXPORT int li_moe_combine(const void* rows, int dtype, const int* place_of, const float* weights, int T, int top, int H, void* y,
                             cudaStream_t stream) {
    LI_REQUIRE(T >= 0 && top > 0 && H > 0, "moe_combine: bad sizes");
    LI_REQUIRE(dtype == LI_F32 || dtype == LI_BF16, "moe_combine: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t e;
    if (dtype == LI_F32)
        e = li_launch_pdl(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)rows, place_of, weights, top, H, (float*)y);
    else
        e = li_launch_pdl(moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)rows, place_of, weights, top, H, (bf16*)y);
    if (e != cudaSuccess) return li_fail("moe_combine: launch failed: %s", cudaGetErrorString(e));
    return li_check_launch("moe_combine");
}
