// Attention through a shared latent: every position keeps ONE row  [c (rank) | k_rot (rot)]  for all heads, where
// c is the normed latent that keys and values are made from and k_rot a rotated key part that all heads share.
// With per-head matrices U_k (unrotated keys from c) and U_v (values from c), a head's score against position j is
//     (q_n . U_k c_j + q_r . k_rot_j) * scale  =  ((U_k^T q_n) . c_j + q_r . k_rot_j) * scale ,
// and its output  U_v (sum_j p_j c_j).  So the query side is first carried into the latent (a product outside this
// file), attention runs over the cached rows as they are, with the first `rank` entries of a row as its value, and
// the per-head value matrix is applied afterwards.
//
// Two kernels:
//   prepare: from the packed projection row  [q latent (q_rank) | kv latent (rank) | shared key part (rot)]  it writes
//            the normed q latent (input of the next projection) and the position's cache row: the normed kv latent
//            and the rotated shared key part.  Norms: x / sqrt(mean(x^2) + eps) * w, 32-bit.
//   attend (exact): one warp per (token, head); the query is [carried part (rank) | rotated part (rot)], the rotation
//            of the query's own part is done here; keys in blocks of 32 from the first visible one's block upward with
//            a running maximum and sum, all 32-bit.  The order of operations for a (token, head) depends only on its
//            own position and window: results are bit-equal however the tokens are cut into steps or batched.
//
// Rotation: the first `rot_dims` entries of the rotated part turn, entry i paired with i + rot_dims/2, by the angle
// whose cosine and sine (already times any magnitude factor) stand in the tables [position, rot_dims/2]; the rest of
// the part passes unchanged.
// Window: position i sees j with 0 <= i - j < window (window 0: all j <= i).

#include "common.cuh"

namespace {

constexpr int PREP_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) latent_prepare_kernel(
    const T* __restrict__ proj, const float* __restrict__ w_q, const float* __restrict__ w_kv, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ slots, const int* __restrict__ block_table,
    T* __restrict__ q_latent, T* __restrict__ pages, int q_rank, int rank, int rot, int rot_dims, int max_pages,
    int page_size) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * (q_rank + rank + rot);
    // the q latent
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += PREP_THREADS) {
        const float v = to_float(row[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    float r = 1.f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += PREP_THREADS)
        q_latent[(size_t)t * q_rank + i] = from_float<T>(to_float(row[i]) * r * w_q[i]);
    if (pages == nullptr) return;
    // the cache row
    const int pos = tok_pos[t];
    const int page = block_table[(size_t)slots[tok_seq[t]] * max_pages + pos / page_size];
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * (rank + rot);
    const T* kv = row + q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += PREP_THREADS) {
        const float v = to_float(kv[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    r = 1.f / sqrtf(ss / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += PREP_THREADS) dst[i] = from_float<T>(to_float(kv[i]) * r * w_kv[i]);
    const int half = rot_dims >> 1;
    const T* kr = kv + rank;
    for (int i = threadIdx.x; i < rot; i += PREP_THREADS) {
        float v = to_float(kr[i]);
        if (i < rot_dims) {
            const int f = i < half ? i : i - half;
            const float c = cos_table[(size_t)pos * half + f], s = sin_table[(size_t)pos * half + f];
            const float other = to_float(kr[i < half ? i + half : i - half]);
            v = i < half ? v * c - other * s : v * c + other * s;
        }
        dst[rank + i] = from_float<T>(v);
    }
}

constexpr int WARPS = 4;
constexpr int MAX_ACC = 32;  // rank <= 1024

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int d);
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; ++i) acc = fmaf(q[i], k[i], acc);
    return acc;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; ++i) acc = fmaf(q[i], __bfloat162float(k[i]), acc);
    return acc;
}

// q_carried: [token, head, rank] with the given strides (elements); q_raw: [token, head, q_raw_dim] with the head's
// rotated part at q_rot_at; out: [token, head, rank] with the given strides.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32) attention_latent_exact_kernel(
    const T* __restrict__ q_carried, long long qc_tok, long long qc_head, const T* __restrict__ q_raw, int q_raw_dim,
    int q_rot_at, const float* __restrict__ cos_table, const float* __restrict__ sin_table, const T* __restrict__ pages,
    T* __restrict__ out, long long out_tok, long long out_head, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ slots, const int* __restrict__ block_table, int n_tokens,
    int n_heads, int rank, int rot, int rot_dims, int max_pages, int page_size, float scale, int window) {
    extern __shared__ float q_smem[];  // WARPS * (rank + rot)
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * WARPS + warp;
    if (wid >= (long long)n_tokens * n_heads) return;  // whole warp leaves together; no block-wide sync below
    const int t = (int)(wid / n_heads);
    const int h = (int)(wid - (long long)t * n_heads);
    const int pos = tok_pos[t];
    const int* table = block_table + (size_t)slots[tok_seq[t]] * max_pages;
    const int width = rank + rot;
    float* qs = q_smem + warp * width;
    const T* qc = q_carried + (size_t)t * qc_tok + (size_t)h * qc_head;
    for (int i = lane; i < rank; i += 32) qs[i] = to_float(qc[i]);
    const T* qr = q_raw + ((size_t)t * n_heads + h) * q_raw_dim + q_rot_at;
    const int half = rot_dims >> 1;
    for (int i = lane; i < rot; i += 32) {
        float v = to_float(qr[i]);
        if (i < rot_dims) {
            const int f = i < half ? i : i - half;
            const float c = cos_table[(size_t)pos * half + f], s = sin_table[(size_t)pos * half + f];
            const float other = to_float(qr[i < half ? i + half : i - half]);
            v = i < half ? v * c - other * s : v * c + other * s;
        }
        qs[rank + i] = v;
    }
    __syncwarp();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_ACC];
#pragma unroll
    for (int c = 0; c < MAX_ACC; ++c) acc[c] = 0.f;
    const int n_acc = (rank + 31) >> 5;

    for (int j0 = (lo >> 5) << 5; j0 <= pos; j0 += 32) {
        const int page = table[j0 / page_size];  // page_size is a multiple of 32: one page per block of keys
        const size_t base = ((size_t)page * page_size + j0 % page_size) * width;
        const int j = j0 + lane;
        const bool valid = j <= pos && j >= lo;
        float s = -INFINITY;
        if (valid) s = dot_row<T>(qs, pages + base + (size_t)lane * width, width) * scale;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        const int first = max(lo - j0, 0), n_here = min(32, pos - j0 + 1);
#pragma unroll
        for (int c = 0; c < MAX_ACC; ++c)
            if (c < n_acc) acc[c] *= corr;
        for (int jj = first; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vrow = pages + base + (size_t)jj * width;
#pragma unroll
            for (int c = 0; c < MAX_ACC; ++c) {
                const int dim = lane + 32 * c;
                if (c < n_acc && dim < rank) acc[c] = fmaf(pj, to_float(vrow[dim]), acc[c]);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)t * out_tok + (size_t)h * out_head;
#pragma unroll
    for (int c = 0; c < MAX_ACC; ++c) {
        const int dim = lane + 32 * c;
        if (c < n_acc && dim < rank) orow[dim] = from_float<T>(acc[c] / l);
    }
}

}  // namespace

GK_EXPORT int gk_latent_prepare(const void* proj, int dtype, const float* w_q, const float* w_kv, float eps,
                                const float* cos_table, const float* sin_table, const int* tok_pos, const int* tok_seq,
                                const int* slots, const int* block_table, void* q_latent, void* pages, int n_tokens,
                                int q_rank, int rank, int rot, int rot_dims, int max_pages, int page_size, int max_position,
                                int table_rows, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "latent_prepare: bad dtype %d", dtype);
    GK_REQUIRE(n_tokens >= 0 && q_rank > 0 && rank > 0 && rot >= 0, "latent_prepare: bad sizes");
    GK_REQUIRE(rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0, "latent_prepare: %d of %d entries cannot turn in pairs",
               rot_dims, rot);
    GK_REQUIRE(rot_dims == 0 || (cos_table && sin_table && table_rows > max_position),
               "latent_prepare: the rotation tables hold %d positions, the step reaches %d", table_rows, max_position);
    GK_REQUIRE(eps > 0.f, "latent_prepare: eps must be positive");
    if (n_tokens == 0) return GK_OK;
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(latent_prepare_kernel<T>, dim3(n_tokens), dim3(PREP_THREADS), 0, (cudaStream_t)stream, (const T*)proj, w_q,
                  w_kv, eps, cos_table, sin_table, tok_pos, tok_seq, slots, block_table, (T*)q_latent, (T*)pages, q_rank, rank,
                  rot, rot_dims, max_pages, page_size);
    })
    GK_CHECK_LAUNCH("latent_prepare");
    return GK_OK;
}

GK_EXPORT int gk_attention_latent_exact(const void* q_carried, long long qc_tok, long long qc_head, const void* q_raw,
                                        int q_raw_dim, int q_rot_at, const float* cos_table, const float* sin_table,
                                        const void* pages, void* out, long long out_tok, long long out_head, int dtype,
                                        const int* tok_pos, const int* tok_seq, const int* slots, const int* block_table,
                                        int n_tokens, int n_heads, int rank, int rot, int rot_dims, int max_pages,
                                        int page_size, float scale, int window, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "attention_latent_exact: bad dtype %d", dtype);
    GK_REQUIRE(n_tokens >= 0 && n_heads > 0 && rank > 0 && rot >= 0, "attention_latent_exact: bad sizes");
    GK_REQUIRE(rank <= 32 * MAX_ACC, "attention_latent_exact: latent size %d is more than %d", rank, 32 * MAX_ACC);
    GK_REQUIRE(rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0, "attention_latent_exact: bad rotation sizes");
    GK_REQUIRE(q_rot_at >= 0 && q_rot_at + rot <= q_raw_dim, "attention_latent_exact: the rotated part lies outside the head");
    GK_REQUIRE(page_size > 0 && page_size % 32 == 0, "attention_latent_exact: page_size %d must be a multiple of 32", page_size);
    GK_REQUIRE(window >= 0, "attention_latent_exact: window must be >= 0 (0 = none)");
    if (n_tokens == 0) return GK_OK;
    const long long warps = (long long)n_tokens * n_heads;
    const long long blocks = (warps + WARPS - 1) / WARPS;
    GK_REQUIRE(blocks < 2147483647LL, "attention_latent_exact: too many tokens");
    const size_t smem = (size_t)WARPS * (rank + rot) * sizeof(float);
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(attention_latent_exact_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, (cudaStream_t)stream,
                  (const T*)q_carried, qc_tok, qc_head, (const T*)q_raw, q_raw_dim, q_rot_at, cos_table, sin_table,
                  (const T*)pages, (T*)out, out_tok, out_head, tok_pos, tok_seq, slots, block_table, n_tokens, n_heads, rank,
                  rot, rot_dims, max_pages, page_size, scale, window);
    })
    GK_CHECK_LAUNCH("attention_latent_exact");
    return GK_OK;
}

// ---- a batch of small products, one per head, for steps of a few tokens:  out[b][m][n] = sum_k x[b][m][k] * w[b][n][k]
// (bfloat16 in, 32-bit sums, rounded once).  x and out are views with batch and row strides (heads lie side by
// side in a token's row); w is contiguous [B, N, K].  One thread per output: with a handful of tokens the products are a
// few hundred kilobytes of weights, read through the L2 once per token, and next to no arithmetic.  (32-bit sums, four
// partial sums an output in a fixed order.)
namespace {

// Four lanes an output: lane q of the quad takes the 8-element pieces q, q + 4, q + 8, ... of the row (all its loads
// independent of one another), and the four partial sums meet by two shuffles in a fixed order.
template <bool VEC>
__global__ void heads_product_kernel(const __nv_bfloat16* __restrict__ x, long long x_batch, long long x_row,
                                     const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long o_batch,
                                     long long o_row, int batch, int m, int n, int k) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 2;
    const int q = threadIdx.x & 3;
    const bool on = idx < (long long)batch * m * n;  // whole quads are on or off; off lanes still take part in the shuffles
    const long long at = on ? idx : 0;
    const int col = (int)(at % n);
    const int tok = (int)((at / n) % m);
    const int b = (int)(at / ((long long)n * m));
    const __nv_bfloat16* xr = x + (size_t)b * x_batch + (size_t)tok * x_row;
    const __nv_bfloat16* wr = w + ((size_t)b * n + col) * k;
    float acc = 0.f;
    if (VEC) {
#pragma unroll 4
        for (int i = q * 8; i < k; i += 32) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xr + i), wv = *reinterpret_cast<const uint4*>(wr + i);
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
            const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float2 xf = __bfloat1622float2(xp[c]), wf = __bfloat1622float2(wp[c]);
                acc = fmaf(xf.x, wf.x, acc);
                acc = fmaf(xf.y, wf.y, acc);
            }
        }
    } else {
#pragma unroll 4
        for (int i = q; i < k; i += 4) acc = fmaf(__bfloat162float(xr[i]), __bfloat162float(wr[i]), acc);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (on && q == 0) out[(size_t)b * o_batch + (size_t)tok * o_row + col] = __float2bfloat16_rn(acc);
}

}  // namespace

GK_EXPORT int gk_heads_product_bf16(const void* x, long long x_batch, long long x_row, const void* w, void* out, long long o_batch,
                                    long long o_row, int batch, int m, int n, int k, void* stream) {
    GK_REQUIRE(batch > 0 && m >= 0 && n > 0 && k > 0, "heads_product: bad sizes batch=%d m=%d n=%d k=%d", batch, m, n, k);
    const long long total = (long long)batch * m * n;
    if (total == 0) return GK_OK;
    const int threads = 128;
    const long long blocks = (total * 4 + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "heads_product: too many outputs");
    const bool vec = k % 8 == 0 && x_batch % 8 == 0 && x_row % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (vec)
        gk_launch(heads_product_kernel<true>, dim3((unsigned)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x, x_batch, x_row,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_batch, o_row, batch, m, n, k);
    else
        gk_launch(heads_product_kernel<false>, dim3((unsigned)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)x, x_batch, x_row,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_batch, o_row, batch, m, n, k);
    GK_CHECK_LAUNCH("heads_product");
    return GK_OK;
}
