// What lies between the q/k(/v) projection and the attention itself, for the attention variants
// the per-head kernel of elementwise.cu does not cover.  One block per token; the token's q and k
// rows pass through shared memory as float32, so a norm may span the whole projection.
//
// In order, per token t at position p of slot s:
//   1. bias:      q += b_q, k += b_k, v += b_v                              (each optional)
//   2. values:    either the row carries v heads of its own, or the values ARE the keys as they
//                 stand after step 1 (before norm and rotation): v_cache[p] = k
//   3. norm:      none | per head: x * rsqrt(mean_head(x^2) + eps) * w[d]
//                      | whole projection: x * rsqrt(mean_row(x^2) + eps) * w[heads * d]
//   4. rotation of the first rot_dim values of every q and k head by the angles of position p:
//                 pairing "half": value i turns with value i + rot_dim/2;
//                 pairing "adjacent": value 2i turns with value 2i + 1;
//                 (a, b) -> (a cos - b sin, b cos + a sin); the table holds (cos, sin) per
//                 position and frequency, already scaled by whatever the encoding prescribes
//   5. q back in place, k into the cache page of (s, p) (and in place if asked)
//   6. the output projection's bias, added to the token's row of the float32 residual stream:
//                 nothing reads that row between the block's norm and the output projection,
//                 which accumulates into it
// A value head has `dv` values, which need not be the keys' `d` (the row is q heads, k heads, then v
// heads of dv values each; the cache's value pages are laid out by dv).
// All arithmetic is float32; storage is float32 or bfloat16.
#include "common.cuh"

#define PREP_THREADS 256
#define PREP_NORM_NONE 0
#define PREP_NORM_HEAD 1
#define PREP_NORM_ROW 2
#define PREP_PAIR_HALF 0
#define PREP_PAIR_ADJACENT 1
#define PREP_WRITE_CACHE 1
#define PREP_K_IN_PLACE 2
#define PREP_VALUES_ARE_KEYS 4

struct PrepArgs {
    long token_stride;
    int n_tokens, n_q, n_kv, d, dv;
    const void *q_bias, *k_bias, *v_bias;
    int bias_dtype;
    const void *q_norm_w, *k_norm_w;
    int norm_dtype, norm_mode;
    float eps;
    const float2* rope_table;
    int rot_dim, table_positions, pairing;
    const int *token_pos, *token_slot;
    void *k_pages, *v_pages;
    const int* block_table;
    int table_stride, flags;
    float* residual;
    long residual_stride;
    const void* out_bias;
    int out_bias_dtype, width;
    int* status;
};

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) qk_prepare_kernel(T* __restrict__ qkv, const PrepArgs a) {
    pdl_trigger();
    extern __shared__ float rowbuf[];             // [(n_q + n_kv) * d] q then k, float32
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int slot = a.token_slot[t];
    if (slot < 0) return;                         // padding row
    const int pos = a.token_pos[t];
    const int d = a.d, nq = a.n_q * d, nk = a.n_kv * d;
    const bool own_v = !(a.flags & PREP_VALUES_ARE_KEYS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = PREP_THREADS / 32;
    int page = -1;
    if (a.flags & PREP_WRITE_CACHE) page = a.block_table[(size_t)slot * a.table_stride + pos / BFI_PAGE_TOKENS];
    const bool bad_pos = a.rope_table != nullptr && (pos < 0 || pos >= a.table_positions);
    pdl_wait();
    T* row = qkv + (size_t)t * a.token_stride;

    // ---- 1. the row with its biases, and the sums of squares of the q and of the k projection
    float ss_q = 0.0f, ss_k = 0.0f;
    for (int j = threadIdx.x; j < nq + nk; j += PREP_THREADS) {
        float v = to_f32(row[j]);
        if (j < nq) {
            if (a.q_bias) v += load_as_f32(a.q_bias, a.bias_dtype, j);
            ss_q = fmaf(v, v, ss_q);
        } else {
            if (a.k_bias) v += load_as_f32(a.k_bias, a.bias_dtype, j - nq);
            ss_k = fmaf(v, v, ss_k);
        }
        rowbuf[j] = v;
    }
    float row_scale_q = 1.0f, row_scale_k = 1.0f;
    if (a.norm_mode == PREP_NORM_ROW) {
        ss_q = block_sum(ss_q, scratch);
        ss_k = block_sum(ss_k, scratch);
        if (nq > 0) row_scale_q = 1.0f / sqrtf(ss_q / (float)nq + a.eps);
        if (nk > 0) row_scale_k = 1.0f / sqrtf(ss_k / (float)nk + a.eps);
    } else {
        __syncthreads();
    }
    if (a.flags & PREP_WRITE_CACHE) {
        if (page < 0) {
            if (threadIdx.x == 0 && a.status && a.n_kv > 0) atomicOr(a.status, BFI_STATUS_NO_PAGE);
        } else {
            // ---- 2. the values: the keys as they stand now, or the row's own v heads
            T* vp = reinterpret_cast<T*>(a.v_pages);
            const int dv = own_v ? a.dv : d;     // values that are the keys have the keys' size
            for (int j = threadIdx.x; j < a.n_kv * dv; j += PREP_THREADS) {
                const int h = j / dv, e = j - h * dv;
                float v;
                if (own_v) {
                    v = to_f32(row[nq + nk + j]);
                    if (a.v_bias) v += load_as_f32(a.v_bias, a.bias_dtype, j);
                } else {
                    v = rowbuf[nq + j];
                }
                vp[(((size_t)page * a.n_kv + h) * BFI_PAGE_TOKENS + (pos % BFI_PAGE_TOKENS)) * dv + e] = from_f32<T>(v);
            }
        }
    }
    __syncthreads();                              // the keys are about to be normalised in place
    if (bad_pos) {
        if (threadIdx.x == 0 && a.status) atomicOr(a.status, BFI_STATUS_BAD_POSITION);
        return;
    }

    // ---- 3. to 5., a warp per head
    const int half = a.rot_dim >> 1;
    const float2* cs = a.rope_table ? a.rope_table + (size_t)pos * half : nullptr;
    for (int hh = warp; hh < a.n_q + a.n_kv; hh += n_warps) {
        const bool is_q = hh < a.n_q;
        float* b = rowbuf + (size_t)hh * d;
        const void* nw = is_q ? a.q_norm_w : a.k_norm_w;
        if (a.norm_mode != PREP_NORM_NONE && nw != nullptr) {
            float scale = is_q ? row_scale_q : row_scale_k;
            int w0 = (is_q ? hh : hh - a.n_q) * d;          // a row norm's weight spans the projection
            if (a.norm_mode == PREP_NORM_HEAD) {
                float ss = 0.0f;
                for (int j = lane; j < d; j += 32) ss = fmaf(b[j], b[j], ss);
                ss = warp_sum(ss);
                scale = 1.0f / sqrtf(ss / (float)d + a.eps);
                w0 = 0;
            }
            for (int j = lane; j < d; j += 32) b[j] = b[j] * scale * load_as_f32(nw, a.norm_dtype, w0 + j);
            __syncwarp();
        }
        T* dst_cache = nullptr;
        if (!is_q && (a.flags & PREP_WRITE_CACHE) && page >= 0)
            dst_cache = reinterpret_cast<T*>(a.k_pages) +
                        (((size_t)page * a.n_kv + (hh - a.n_q)) * BFI_PAGE_TOKENS + (pos % BFI_PAGE_TOKENS)) * d;
        T* dst_row = (is_q || (a.flags & PREP_K_IN_PLACE)) ? row + (size_t)hh * d : nullptr;
        if (cs != nullptr) {
            for (int i = lane; i < half; i += 32) {
                const int i0 = a.pairing == PREP_PAIR_HALF ? i : 2 * i;
                const int i1 = a.pairing == PREP_PAIR_HALF ? i + half : 2 * i + 1;
                const float2 c = cs[i];
                const float x0 = b[i0], x1 = b[i1];
                const float o0 = x0 * c.x - x1 * c.y;
                const float o1 = x1 * c.x + x0 * c.y;
                if (dst_row) dst_row[i0] = from_f32<T>(o0), dst_row[i1] = from_f32<T>(o1);
                if (dst_cache) dst_cache[i0] = from_f32<T>(o0), dst_cache[i1] = from_f32<T>(o1);
            }
        }
        for (int j = (cs ? a.rot_dim : 0) + lane; j < d; j += 32) {
            if (dst_row) dst_row[j] = from_f32<T>(b[j]);
            if (dst_cache) dst_cache[j] = from_f32<T>(b[j]);
        }
    }

    // ---- 6. the output projection's bias goes to the residual row now
    if (a.out_bias != nullptr) {
        float* r = a.residual + (size_t)t * a.residual_stride;
        for (int j = threadIdx.x; j < a.width; j += PREP_THREADS) r[j] += load_as_f32(a.out_bias, a.out_bias_dtype, j);
    }
}

extern "C" int bfi_qk_prepare(void* qkv, int dtype, long token_stride, int n_tokens, int n_q, int n_kv, int d, int dv,
                              const void* q_bias, const void* k_bias, const void* v_bias, int bias_dtype,
                              const void* q_norm_w, const void* k_norm_w, int norm_dtype, int norm_mode, float eps,
                              const void* rope_table, int rot_dim, int table_positions, int pairing,
                              const int* token_pos, const int* token_slot, void* k_pages, void* v_pages,
                              const int* block_table, int table_stride, int flags, float* residual,
                              long residual_stride, const void* out_bias, int out_bias_dtype, int width, int* status,
                              cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(norm_dtype) && dtype_ok(bias_dtype) && dtype_ok(out_bias_dtype),
                "qk_prepare: unknown dtype code");
    BFI_REQUIRE(n_tokens >= 0 && n_q >= 0 && n_kv >= 0 && n_q + n_kv > 0, "qk_prepare: bad head counts q=%d kv=%d", n_q, n_kv);
    BFI_REQUIRE(d > 0 && d % 2 == 0, "qk_prepare: head_dim %d must be even", d);
    BFI_REQUIRE(norm_mode >= PREP_NORM_NONE && norm_mode <= PREP_NORM_ROW, "qk_prepare: unknown norm mode %d", norm_mode);
    BFI_REQUIRE(pairing == PREP_PAIR_HALF || pairing == PREP_PAIR_ADJACENT, "qk_prepare: unknown pairing %d", pairing);
    const bool own_v = !(flags & PREP_VALUES_ARE_KEYS);
    BFI_REQUIRE(dv > 0 && (own_v || dv == d), "qk_prepare: value size %d (values that are the keys have the keys' size %d)", dv, d);
    BFI_REQUIRE(token_stride >= (long)(n_q + n_kv) * d + (own_v ? (long)n_kv * dv : 0), "qk_prepare: token stride shorter than the heads");
    if (rope_table) {
        BFI_REQUIRE(rot_dim > 0 && rot_dim % 2 == 0 && rot_dim <= d,
                    "qk_prepare: rotary width %d must be even and at most head_dim %d", rot_dim, d);
        BFI_REQUIRE(table_positions > 0, "qk_prepare: empty rotation table");
    }
    if ((flags & PREP_WRITE_CACHE) && n_kv > 0)
        BFI_REQUIRE(k_pages && v_pages && block_table && table_stride > 0, "qk_prepare: cache write without a cache");
    if (out_bias) BFI_REQUIRE(residual && width > 0 && residual_stride >= width, "qk_prepare: output bias without a residual row");
    if (n_tokens == 0) return 0;
    const size_t smem = (size_t)(n_q + n_kv) * d * sizeof(float);
    BFI_REQUIRE(smem <= 200 * 1024, "qk_prepare: %d values of q and k per token do not fit shared memory", (n_q + n_kv) * d);
    PrepArgs a;
    a.token_stride = token_stride, a.n_tokens = n_tokens, a.n_q = n_q, a.n_kv = n_kv, a.d = d, a.dv = dv;
    a.q_bias = q_bias, a.k_bias = k_bias, a.v_bias = v_bias, a.bias_dtype = bias_dtype;
    a.q_norm_w = q_norm_w, a.k_norm_w = k_norm_w, a.norm_dtype = norm_dtype, a.norm_mode = norm_mode, a.eps = eps;
    a.rope_table = (const float2*)rope_table, a.rot_dim = rot_dim, a.table_positions = table_positions, a.pairing = pairing;
    a.token_pos = token_pos, a.token_slot = token_slot, a.k_pages = k_pages, a.v_pages = v_pages;
    a.block_table = block_table, a.table_stride = table_stride, a.flags = flags;
    a.residual = residual, a.residual_stride = residual_stride, a.out_bias = out_bias, a.out_bias_dtype = out_bias_dtype;
    a.width = width, a.status = status;
    cudaError_t e = cudaSuccess;
    if (dtype == BFI_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(qk_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) bfi_launch(qk_prepare_kernel<float>, dim3(n_tokens), dim3(PREP_THREADS), smem, stream, (float*)qkv, a);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(qk_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) bfi_launch(qk_prepare_kernel<bf16>, dim3(n_tokens), dim3(PREP_THREADS), smem, stream, (bf16*)qkv, a);
    }
    if (e != cudaSuccess) return bfi_fail("qk_prepare: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    return bfi_check_launch("qk_prepare");
}

BFI_TRACE_EXPORT(attention_prepare)
