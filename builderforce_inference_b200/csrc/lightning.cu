// Linear attention with a per-head decay ("lightning attention"), the general kernels: any sizes,
// any step shape (whole prompts, continuations, single tokens), float32 or bfloat16 storage of
// the projections, float32 arithmetic and float32 state.
//
// Per sequence and head, with q_t, k_t (D values) and v_t (V values) the activated projections:
//     S_t = decay * S_(t-1) + k_t v_t^T          S is D x V, float32, kept per slot between steps
//     o_t = S_t^T q_t
// Column c of S, and with it value c of o, depends on no other column, so a block owns a range of
// `vb` columns of one head of one sequence and walks the sequence's new tokens in order.  Thread
// (g, c) of a block holds rows g, g + groups, ... of column c in shared memory.
//
// After the recurrence the heads of a token are normalised together and gated:
//     y = o * rsqrt(mean(o^2) + eps) * w * sigmoid(gate)        (bfi_gated_rmsnorm)
#include "common.cuh"

#define LIGHT_ACT_NONE 0
#define LIGHT_ACT_SILU 1

__device__ __forceinline__ float light_silu(float x) {
    float s;
    if (x >= 0.0f) {
        s = 1.0f / (1.0f + expf(-x));
    } else {
        const float z = expf(x);
        s = z / (1.0f + z);
    }
    return x * s;
}
__device__ __forceinline__ float light_sigmoid(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float z = expf(x);
    return z / (1.0f + z);
}

template <typename T>
__global__ void lightning_scan_kernel(const T* __restrict__ proj, long stride, int q_off, int k_off, int v_off,
                                      float* __restrict__ out, long out_stride, float* __restrict__ state,
                                      const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
                                      const int* __restrict__ seq_slot, int H, int D, int V, int vb, int v_blocks,
                                      int act) {
    pdl_trigger();
    extern __shared__ float sm[];
    float* S = sm;                     // [D][vb]
    float* qs = S + (size_t)D * vb;    // [D]
    float* ks = qs + D;                // [D]
    float* red = ks + D;               // [threads]
    const int seq = blockIdx.y;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int h = blockIdx.x / v_blocks;
    const int v0 = (blockIdx.x - h * v_blocks) * vb;
    const int t0 = cu_seqlens[seq], nt = cu_seqlens[seq + 1] - t0;
    const int c = threadIdx.x % vb, g = threadIdx.x / vb, ng = blockDim.x / vb;
    const bool col_ok = v0 + c < V;
    const float w = decay[h];
    // the state of earlier steps (zeroed when the slot was taken) does not come from this step's kernels
    float* sp = state + (((size_t)slot * H + h) * D) * V + v0;
    for (int d = g; d < D; d += ng) S[d * vb + c] = col_ok ? sp[(size_t)d * V + c] : 0.0f;
    pdl_wait();
    for (int t = 0; t < nt; ++t) {
        const T* row = proj + (size_t)(t0 + t) * stride + (size_t)h * D;
        for (int j = threadIdx.x; j < D; j += blockDim.x) {
            const float qv = to_f32(row[q_off + j]), kv = to_f32(row[k_off + j]);
            qs[j] = act == LIGHT_ACT_SILU ? light_silu(qv) : qv;
            ks[j] = act == LIGHT_ACT_SILU ? light_silu(kv) : kv;
        }
        float vv = 0.0f;
        if (col_ok) {
            vv = to_f32(proj[(size_t)(t0 + t) * stride + v_off + (size_t)h * V + v0 + c]);
            if (act == LIGHT_ACT_SILU) vv = light_silu(vv);
        }
        __syncthreads();
        float acc = 0.0f;
        for (int d = g; d < D; d += ng) {
            const float s = fmaf(w, S[d * vb + c], ks[d] * vv);
            S[d * vb + c] = s;
            acc = fmaf(s, qs[d], acc);
        }
        red[threadIdx.x] = acc;
        __syncthreads();
        if (threadIdx.x < vb && col_ok) {
            float o = 0.0f;
            for (int i = 0; i < ng; ++i) o += red[i * vb + threadIdx.x];
            out[(size_t)(t0 + t) * out_stride + (size_t)h * V + v0 + c] = o;
        }
    }
    if (col_ok)
        for (int d = g; d < D; d += ng) sp[(size_t)d * V + c] = S[d * vb + c];
}

// One new token per sequence: the state never rests in shared memory.  A block owns 32 columns of
// one head of one sequence; thread (g, c) holds rows g, g + 8, ... of column c in registers, all of
// them asked for before the wait for the kernel that makes q, k and v (the state was left by an
// earlier step), so that a step's traffic, which is the states read and written once, streams.
#define LIGHT_STEP_COLS 32
#define LIGHT_STEP_GROUPS 8

template <typename T, int RPT>
__global__ void __launch_bounds__(LIGHT_STEP_COLS * LIGHT_STEP_GROUPS)
lightning_step_kernel(const T* __restrict__ proj, long stride, int q_off, int k_off, int v_off, float* __restrict__ out,
                      long out_stride, float* __restrict__ state, const float* __restrict__ decay,
                      const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, int H, int D, int V,
                      int v_blocks, int act) {
    pdl_trigger();
    __shared__ float qs[LIGHT_STEP_GROUPS * RPT], ks[LIGHT_STEP_GROUPS * RPT];
    __shared__ float red[LIGHT_STEP_GROUPS][LIGHT_STEP_COLS];
    const int seq = blockIdx.y;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int h = blockIdx.x / v_blocks;
    const int v0 = (blockIdx.x - h * v_blocks) * LIGHT_STEP_COLS;
    const int c = threadIdx.x & (LIGHT_STEP_COLS - 1), g = threadIdx.x / LIGHT_STEP_COLS;
    const bool col_ok = v0 + c < V;
    const float w = decay[h];
    float* sp = state + (((size_t)slot * H + h) * D) * V + v0 + c;
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int d = g + LIGHT_STEP_GROUPS * i;
        S[i] = (col_ok && d < D) ? sp[(size_t)d * V] : 0.0f;
    }
    pdl_wait();
    const int t = cu_seqlens[seq];
    const T* row = proj + (size_t)t * stride;
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        const float qv = to_f32(row[q_off + (size_t)h * D + j]), kv = to_f32(row[k_off + (size_t)h * D + j]);
        qs[j] = act == LIGHT_ACT_SILU ? light_silu(qv) : qv;
        ks[j] = act == LIGHT_ACT_SILU ? light_silu(kv) : kv;
    }
    float vv = 0.0f;
    if (col_ok) {
        vv = to_f32(row[v_off + (size_t)h * V + v0 + c]);
        if (act == LIGHT_ACT_SILU) vv = light_silu(vv);
    }
    __syncthreads();
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int d = g + LIGHT_STEP_GROUPS * i;
        if (d < D) {
            const float s = fmaf(w, S[i], ks[d] * vv);
            if (col_ok) sp[(size_t)d * V] = s;
            acc = fmaf(s, qs[d], acc);
        }
    }
    red[g][c] = acc;
    __syncthreads();
    if (g == 0 && col_ok) {
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < LIGHT_STEP_GROUPS; ++i) o += red[i][c];
        out[(size_t)t * out_stride + (size_t)h * V + v0 + c] = o;
    }
}

template <typename T>
static bool launch_light_step(const void* proj, long stride, int q_off, int k_off, int v_off, float* out, long out_stride,
                              float* state, const float* decay, const int* cu_seqlens, const int* seq_slot, int n_seqs,
                              int H, int D, int V, int act, cudaStream_t stream) {
    const int v_blocks = (V + LIGHT_STEP_COLS - 1) / LIGHT_STEP_COLS;
    const dim3 grid(H * v_blocks, n_seqs), block(LIGHT_STEP_COLS * LIGHT_STEP_GROUPS);
#define BFI_LIGHT_STEP(R)                                                                                              \
    bfi_launch(lightning_step_kernel<T, R>, grid, block, 0, stream, (const T*)proj, stride, q_off, k_off, v_off, out,  \
               out_stride, state, decay, cu_seqlens, seq_slot, H, D, V, v_blocks, act)
    if (D <= 32) BFI_LIGHT_STEP(4);
    else if (D <= 64) BFI_LIGHT_STEP(8);
    else if (D <= 128) BFI_LIGHT_STEP(16);
    else if (D <= 256) BFI_LIGHT_STEP(32);
    else return false;
#undef BFI_LIGHT_STEP
    return true;
}

extern "C" int bfi_lightning_scan(const void* proj, int dtype, long stride, int q_off, int k_off, int v_off, float* out,
                                  long out_stride, float* state, const float* decay, const int* cu_seqlens,
                                  const int* seq_slot, int n_seqs, int H, int D, int V, int act, int few_tokens,
                                  cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "lightning_scan: unknown dtype code %d", dtype);
    BFI_REQUIRE(H > 0 && D > 0 && V > 0, "lightning_scan: bad sizes heads=%d dim=%d vdim=%d", H, D, V);
    BFI_REQUIRE(act == LIGHT_ACT_NONE || act == LIGHT_ACT_SILU, "lightning_scan: unknown activation %d", act);
    BFI_REQUIRE(out_stride >= (long)H * V, "lightning_scan: output stride shorter than the heads");
    if (n_seqs <= 0) return 0;
    if (few_tokens == 2 && n_seqs <= 65535) {      // every sequence brings exactly one token: the state stays in registers
        const bool ran = dtype == BFI_F32
            ? launch_light_step<float>(proj, stride, q_off, k_off, v_off, out, out_stride, state, decay, cu_seqlens, seq_slot, n_seqs, H, D, V, act, stream)
            : launch_light_step<bf16>(proj, stride, q_off, k_off, v_off, out, out_stride, state, decay, cu_seqlens, seq_slot, n_seqs, H, D, V, act, stream);
        if (ran) return bfi_check_launch("lightning_step");
    }
    // columns per block: few where the step is short (more blocks share the state's traffic)
    int vb = V;
    const int want = few_tokens ? 32 : 64;
    if (V > want) vb = want;
    BFI_REQUIRE(vb <= 1024, "lightning_scan: value size %d too large", V);
    const int v_blocks = (V + vb - 1) / vb;
    int threads = vb * (256 / vb > 0 ? 256 / vb : 1);
    if (threads < 32) threads = vb * ((32 + vb - 1) / vb);
    BFI_REQUIRE((long)H * v_blocks <= 2147483647L && n_seqs <= 65535, "lightning_scan: too many heads or sequences for one launch");
    const size_t smem = ((size_t)D * vb + 2 * (size_t)D + threads) * sizeof(float);
    BFI_REQUIRE(smem <= 200 * 1024, "lightning_scan: a state tile of %d x %d does not fit shared memory", D, vb);
    cudaError_t e = cudaSuccess;
    if (dtype == BFI_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(lightning_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(lightning_scan_kernel<float>, dim3(H * v_blocks, n_seqs), dim3(threads), smem, stream, (const float*)proj,
                       stride, q_off, k_off, v_off, out, out_stride, state, decay, cu_seqlens, seq_slot, H, D, V, vb, v_blocks, act);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(lightning_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            bfi_launch(lightning_scan_kernel<bf16>, dim3(H * v_blocks, n_seqs), dim3(threads), smem, stream, (const bf16*)proj,
                       stride, q_off, k_off, v_off, out, out_stride, state, decay, cu_seqlens, seq_slot, H, D, V, vb, v_blocks, act);
    }
    if (e != cudaSuccess) return bfi_fail("lightning_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("lightning_scan");
}

// ------------------------------------------------------------------------------------------
// y[t, :] = x[t, :] * rsqrt(mean(x[t, :]^2) + eps) * w * sigmoid(gate[t, :])
// x float32 (the recurrence's output), gate and y in the activation storage type.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ x, long x_stride, const T* __restrict__ gate, long gate_stride,
                                     const void* __restrict__ w, int w_dtype, T* __restrict__ y, long y_stride, int width,
                                     float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* xr = x + (size_t)t * x_stride;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) ss = fmaf(xr[j], xr[j], ss);
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    const T* gr = gate + (size_t)t * gate_stride;
    T* yr = y + (size_t)t * y_stride;
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        yr[j] = from_f32<T>(xr[j] * scale * load_as_f32(w, w_dtype, j) * light_sigmoid(to_f32(gr[j])));
}

extern "C" int bfi_gated_rmsnorm(const float* x, long x_stride, const void* gate, long gate_stride, int dtype, const void* w,
                                 int w_dtype, void* y, long y_stride, int n_rows, int width, float eps, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(w_dtype), "gated_rmsnorm: unknown dtype code");
    BFI_REQUIRE(n_rows >= 0 && width > 0, "gated_rmsnorm: bad sizes rows=%d width=%d", n_rows, width);
    BFI_REQUIRE(x_stride >= width && gate_stride >= width && y_stride >= width, "gated_rmsnorm: row stride shorter than the row");
    if (n_rows == 0) return 0;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == BFI_F32)
        bfi_launch(gated_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, x_stride, (const float*)gate, gate_stride, w,
                   w_dtype, (float*)y, y_stride, width, eps);
    else
        bfi_launch(gated_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, x_stride, (const bf16*)gate, gate_stride, w,
                   w_dtype, (bf16*)y, y_stride, width, eps);
    return bfi_check_launch("gated_rmsnorm");
}

BFI_TRACE_EXPORT(lightning)
