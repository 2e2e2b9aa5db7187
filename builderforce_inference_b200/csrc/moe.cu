// A routed feed-forward (mixture of experts): the router's decision and the experts' products for
// the (token, chosen expert) pairs, reading only the chosen experts' weights.  Float32 or
// bfloat16 storage of activations and expert weights, float32 arithmetic everywhere.
//
// bfi_moe_route, per token with router logits z[0..E) (float32):
//     s = softmax(z);  choice_e = s_e + correction_e
//     experts form `n_groups` equal groups of neighbours; a group's score is its largest choice
//     score; only experts of the `keep` best groups can be chosen (the others count as minus
//     infinity); the `top` largest choice scores among them are chosen, the lowest index winning
//     a tie; the weights are the chosen experts' s (not renormalised) times `weight_scale`.
//     With `extra` (a logit beside the experts', column E of z) gate[t] = sigmoid(z_E): the factor
//     of an expert that every token uses.
// bfi_moe_gate_up:  act[t, k, :] = silu(W_gate[e] h_t) * (W_up[e] h_t),  e = idx[t, k]
// bfi_moe_down:     out[t, :] (= | +=) sum_k weight[t, k] * W_down[idx[t, k]] act[t, k, :]
//                                      + gate[t] * shared[t, :]            (the last term optional)
#include "common.cuh"

__device__ __forceinline__ float moe_sigmoid(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}

// One warp per token.  Shared memory per warp: s[E], choice[E], group[n_groups].
__global__ void moe_route_kernel(const float* __restrict__ z, long z_stride, const float* __restrict__ correction,
                                 int* __restrict__ idx, float* __restrict__ weight, float* __restrict__ gate,
                                 int n_tokens, int E, int top, int n_groups, int keep, float weight_scale, int extra) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int t = blockIdx.x * n_warps + warp;
    if (t >= n_tokens) return;
    float* s = sm + (size_t)warp * (2 * E + n_groups);
    float* choice = s + E;
    float* gs = choice + E;
    const float* zr = z + (size_t)t * z_stride;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
    m = warp_max(m);
    float sum = 0.0f;
    for (int e = lane; e < E; e += 32) {
        const float p = expf(zr[e] - m);
        s[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        s[e] *= inv;
        choice[e] = s[e] + (correction ? correction[e] : 0.0f);
    }
    __syncwarp();
    const int per = E / n_groups;
    if (n_groups > 1 && keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, choice[e]);
            gs[g] = best;
        }
        __syncwarp();
        // the `keep` best groups are marked by +inf in gs, one per round
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gs[g];
                if (v != INFINITY && (v > best || (v == best && g < at))) best = v, at = g;
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
            }
            if (lane == 0 && at != 0x7fffffff) gs[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    for (int r = 0; r < top; ++r) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = choice[e];
            if (!isnan(v) && (v > best || (v == best && e < at))) best = v, at = e;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
        }
        if (at == 0x7fffffff) at = 0;                  // nothing left to choose from: expert 0 with weight 0
        if (lane == 0) {
            idx[(size_t)t * top + r] = at;
            weight[(size_t)t * top + r] = best == -INFINITY ? 0.0f : s[at] * weight_scale;
            choice[at] = NAN;                          // taken
        }
        __syncwarp();
    }
    if (extra && lane == 0) gate[t] = moe_sigmoid(zr[E]);
}

extern "C" int bfi_moe_route(const float* z, long z_stride, const float* correction, int* idx, float* weight, float* gate,
                             int n_tokens, int E, int top, int n_groups, int keep, float weight_scale, int extra,
                             cudaStream_t stream) {
    BFI_REQUIRE(E > 0 && top > 0 && top <= E, "moe_route: cannot choose %d of %d experts", top, E);
    BFI_REQUIRE(n_groups > 0 && E % n_groups == 0 && keep > 0 && keep <= n_groups,
                "moe_route: %d experts in %d groups, %d kept", E, n_groups, keep);
    BFI_REQUIRE((long)keep * (E / n_groups) >= top, "moe_route: %d groups of %d experts cannot give %d", keep, E / n_groups, top);
    BFI_REQUIRE(z_stride >= E + (extra ? 1 : 0), "moe_route: a row of logits is shorter than the experts");
    BFI_REQUIRE(!extra || gate != nullptr, "moe_route: the extra logit needs a place for its gate");
    if (n_tokens <= 0) return 0;
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + n_groups) * sizeof(float);
    BFI_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts are too many for this kernel", E);
    bfi_launch(moe_route_kernel, dim3((n_tokens + warps - 1) / warps), dim3(32 * warps), smem, stream, z, z_stride, correction,
               idx, weight, gate, n_tokens, E, top, n_groups, keep, weight_scale, extra);
    return bfi_check_launch("moe_route");
}

// dot of a weight row (storage T) with a float32 vector in shared memory, across a warp
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ x, int n, int lane);

template <>
__device__ __forceinline__ float warp_dot<float>(const float* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.0f;
    if ((n & 3) == 0 && ((uintptr_t)w & 15) == 0) {
        for (int j = lane * 4; j < n; j += 128) {
            const float4 a = *reinterpret_cast<const float4*>(w + j);
            acc = fmaf(a.x, x[j], acc), acc = fmaf(a.y, x[j + 1], acc), acc = fmaf(a.z, x[j + 2], acc), acc = fmaf(a.w, x[j + 3], acc);
        }
    } else {
        for (int j = lane; j < n; j += 32) acc = fmaf(w[j], x[j], acc);
    }
    return warp_sum(acc);
}
template <>
__device__ __forceinline__ float warp_dot<bf16>(const bf16* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.0f;
    if ((n & 7) == 0 && ((uintptr_t)w & 15) == 0) {
        for (int j = lane * 8; j < n; j += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + j);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                acc = fmaf(f.x, x[j + 2 * i], acc), acc = fmaf(f.y, x[j + 2 * i + 1], acc);
            }
        }
    } else {
        for (int j = lane; j < n; j += 32) acc = fmaf(__bfloat162float(w[j]), x[j], acc);
    }
    return warp_sum(acc);
}

#define MOE_WARPS 8

// grid (pairs, chunks of ff rows); W_gate, W_up: [E][ff][width]
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_gate_up_kernel(const T* __restrict__ h, long h_stride, const T* __restrict__ w_gate, const T* __restrict__ w_up,
                   const int* __restrict__ idx, const int* __restrict__ token_slot, T* __restrict__ act, int top,
                   int width, int ff, int rows_per_block) {
    pdl_trigger();
    extern __shared__ float hs[];                  // [width]
    const int pair = blockIdx.x;
    const int t = pair / top;
    if (token_slot[t] < 0) return;                 // padding row
    pdl_wait();
    const int e = idx[pair];
    for (int j = threadIdx.x; j < width; j += blockDim.x) hs[j] = to_f32(h[(size_t)t * h_stride + j]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r0 = blockIdx.y * rows_per_block;
    const int r1 = min(ff, r0 + rows_per_block);
    for (int r = r0 + warp; r < r1; r += MOE_WARPS) {
        const size_t off = ((size_t)e * ff + r) * width;
        const float g = warp_dot<T>(w_gate + off, hs, width, lane);
        const float u = warp_dot<T>(w_up + off, hs, width, lane);
        if (lane == 0) act[(size_t)pair * ff + r] = from_f32<T>(g * moe_sigmoid(g) * u);
    }
}

extern "C" int bfi_moe_gate_up(const void* h, long h_stride, int dtype, const void* w_gate, const void* w_up,
                               const int* idx, const int* token_slot, void* act, int n_tokens, int top, int width, int ff,
                               cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "moe_gate_up: unknown dtype code %d", dtype);
    BFI_REQUIRE(top > 0 && width > 0 && ff > 0 && h_stride >= width, "moe_gate_up: bad sizes");
    if (n_tokens <= 0) return 0;
    const long pairs = (long)n_tokens * top;
    BFI_REQUIRE(pairs <= 2147483647L, "moe_gate_up: too many (token, expert) pairs");
    BFI_REQUIRE((size_t)width * 4 <= 160 * 1024, "moe_gate_up: a row of %d values does not fit shared memory", width);
    // enough blocks to fill the device when pairs are few, whole experts per block when they are many
    int chunks = 1;
    const int sms = bfi_sm_count();
    while (pairs * chunks < 4L * sms && chunks * MOE_WARPS < ff) chunks *= 2;
    const int rows_per_block = (ff + chunks - 1) / chunks;
    chunks = (ff + rows_per_block - 1) / rows_per_block;
    const size_t smem = (size_t)width * sizeof(float);
    const dim3 grid((unsigned)pairs, chunks);
    cudaError_t e = cudaSuccess;
    if (dtype == BFI_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_gate_up_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_gate_up_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)h, h_stride,
                       (const float*)w_gate, (const float*)w_up, idx, token_slot, (float*)act, top, width, ff, rows_per_block);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_gate_up_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_gate_up_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)h, h_stride,
                       (const bf16*)w_gate, (const bf16*)w_up, idx, token_slot, (bf16*)act, top, width, ff, rows_per_block);
    }
    if (e != cudaSuccess) return bfi_fail("moe_gate_up: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("moe_gate_up");
}

// grid (tokens, chunks of output columns); W_down: [E][width][ff]
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ idx,
                const float* __restrict__ weight, const int* __restrict__ token_slot, const float* __restrict__ shared_out,
                long shared_stride, const float* __restrict__ gate, float* __restrict__ out, long out_stride, int top,
                int width, int ff, int cols_per_block, int accumulate) {
    pdl_trigger();
    extern __shared__ float as[];                  // [top][ff]
    const int t = blockIdx.x;
    if (token_slot[t] < 0) return;
    pdl_wait();
    for (int j = threadIdx.x; j < top * ff; j += blockDim.x) as[j] = to_f32(act[(size_t)t * top * ff + j]);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c0 = blockIdx.y * cols_per_block;
    const int c1 = min(width, c0 + cols_per_block);
    const float g = gate ? gate[t] : 1.0f;
    for (int c = c0 + warp; c < c1; c += MOE_WARPS) {
        float sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int e = idx[(size_t)t * top + k];
            const float d = warp_dot<T>(w_down + ((size_t)e * width + c) * ff, as + (size_t)k * ff, ff, lane);
            sum = fmaf(weight[(size_t)t * top + k], d, sum);
        }
        if (lane == 0) {
            if (shared_out) sum = fmaf(g, shared_out[(size_t)t * shared_stride + c], sum);
            float* o = out + (size_t)t * out_stride + c;
            *o = accumulate ? *o + sum : sum;
        }
    }
}

extern "C" int bfi_moe_down(const void* act, int dtype, const void* w_down, const int* idx, const float* weight,
                            const int* token_slot, const float* shared_out, long shared_stride, const float* gate,
                            float* out, long out_stride, int n_tokens, int top, int width, int ff, int accumulate,
                            cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "moe_down: unknown dtype code %d", dtype);
    BFI_REQUIRE(top > 0 && width > 0 && ff > 0 && out_stride >= width, "moe_down: bad sizes");
    BFI_REQUIRE(!shared_out || shared_stride >= width, "moe_down: the shared output's rows are shorter than the width");
    if (n_tokens <= 0) return 0;
    const size_t smem = (size_t)top * ff * sizeof(float);
    BFI_REQUIRE(smem <= 160 * 1024, "moe_down: %d x %d activations per token do not fit shared memory", top, ff);
    int chunks = 1;
    const int sms = bfi_sm_count();
    while ((long)n_tokens * chunks < 4L * sms && chunks * MOE_WARPS < width) chunks *= 2;
    const int cols_per_block = (width + chunks - 1) / chunks;
    chunks = (width + cols_per_block - 1) / cols_per_block;
    const dim3 grid(n_tokens, chunks);
    cudaError_t e = cudaSuccess;
    if (dtype == BFI_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_down_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, stream, (const float*)act, (const float*)w_down, idx,
                       weight, token_slot, shared_out, shared_stride, gate, out, out_stride, top, width, ff, cols_per_block, accumulate);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(moe_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(moe_down_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, stream, (const bf16*)act, (const bf16*)w_down, idx,
                       weight, token_slot, shared_out, shared_stride, gate, out, out_stride, top, width, ff, cols_per_block, accumulate);
    }
    if (e != cudaSuccess) return bfi_fail("moe_down: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("moe_down");
}

BFI_TRACE_EXPORT(moe)
