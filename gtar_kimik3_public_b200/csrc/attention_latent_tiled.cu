// Attention over latent rows on the tensor cores (bfloat16 operands, 32-bit scores, softmax and sums): the kernel
// for prompts and for single-token steps of layers that keep one row  [c (rank) | k_rot (rot)]  per position for all
// heads (see attention_latent.cu for the algebra).  All heads read the SAME rows, so a block's sixteen query rows are
// (token, head) pairs of one sequence, head running fastest: with sixteen heads a tile is one token, with four heads
// four consecutive tokens, whose key ranges differ by a few positions only.
//
// A block = one, two or four tiles of 16 query rows, four warps a tile.  Keys come a page (64 positions) at a time through a two-stage cp.async ring;
// rows outside the tile's key range are filled with zeros (a page's unwritten places may hold anything).  Per page:
//   scores:  warp w forms  S[16 x 16 keys 16w..16w+15]  over the whole row width (rank + rot), masks what its rows
//            must not see, and posts its rows' maxima;
//   softmax: with the maxima of all four warps every warp rescales ITS columns of the output, writes its
//            probabilities (bfloat16) into the shared P tile [16 x 64] and posts its partial row sums;
//   output:  warp w adds  P[16 x 64] V[64 x its rank/4 columns]  to its accumulator; V is the first `rank` entries of
//            the same rows, read transposed by ldmatrix.
// So the wide output (rank up to 512) is spread over the warps (64 registers a thread at most) while the scores are
// spread by keys; the P tile and two small arrays of row statistics are what the warps exchange.
//
// Single-token steps have few tiles; `splits` blocks then share a tile's pages and leave partial results
// (maximum, sum, unnormalised output) in scratch, merged by a second kernel in split order.
//
// The query tile is [carried part (rank) | own rotated part (rot)]; the rotation of the own part is done while the
// tile is staged (32-bit, tables of cos and sin).  Sizes: rank a multiple of 64 up to 512, rot a multiple of 16,
// pages of 64 positions.

#include <stdlib.h>

#include "attention_mma.cuh"

namespace {

using namespace attn;

constexpr int COL_WARPS = 4;  // warps that share a 16-row tile: each takes a quarter of a page's keys and of the output's columns
constexpr int P_STRIDE = PAGE + 8;  // bfloat16 elements: 144 bytes a row, so that ldmatrix rows fall into different banks
constexpr float LOG2E = 1.4426950408889634f;

struct TiledArgs {
    const __nv_bfloat16* q_carried; long long qc_tok, qc_head;
    const __nv_bfloat16* q_raw; int q_raw_dim, q_rot_at;
    const float* cos_table; const float* sin_table;
    const __nv_bfloat16* pages;
    __nv_bfloat16* out; long long out_tok, out_head;
    float* part_o; float* part_ml;  // [split, global row, rank] and [split, global row, 2] when splits > 1
    const int* tok_pos; const int* cu_q; const int* slots; const int* block_table;
    int n_heads, rank, rot, rot_dims, max_pages, splits, n_rows_total, window;
    float scale;
};

// NT: 8-column tiles of the output a warp owns at most (rank / 32 <= NT).  MG: 16-row tiles a block holds (1, 2 or 4): its
// 4 * MG warps share every page it loads, so the rows of MG tiles cost one trip of the page from the L2.
template <int NT, int MG>
__global__ void __launch_bounds__(MG * COL_WARPS * 32) attention_latent_tiled_kernel(const TiledArgs a) {
    constexpr int WARPS = MG * COL_WARPS, THREADS = WARPS * 32, ROWS = MG * 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_launch_dependents();
    pdl_wait();
    // the SMs take blocks in index order and a sequence's last tiles have the most keys: those go first
    const int seq = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x, split = blockIdx.z;
    const int first_tok = a.cu_q[seq], n_tok = a.cu_q[seq + 1] - first_tok;
    const int n_rows = n_tok * a.n_heads;
    if (tile * ROWS >= n_rows) return;
    const int width = a.rank + a.rot;
    const int stride = width + 8;  // elements; rows of (width + 8) * 2 bytes: an odd number of 16-byte pieces
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* k_s = q_s + ROWS * stride;                 // two stages of PAGE rows
    __nv_bfloat16* p_s = k_s + 2 * PAGE * stride;             // [ROWS][P_STRIDE]
    float* stat_max = reinterpret_cast<float*>(p_s + ROWS * P_STRIDE);  // [2][MG][COL_WARPS][16]
    float* stat_sum = stat_max + 2 * WARPS * 16;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
    const int mg = warp / COL_WARPS, cg = warp % COL_WARPS;  // which 16-row tile, which quarter of keys and columns

    // ---- the tile's rows: row r is head (r0 + r) % H of token (r0 + r) / H of the sequence's step
    const int r0 = tile * ROWS;
    const int last_row = min(r0 + ROWS, n_rows) - 1;
    const int tok_lo = r0 / a.n_heads, tok_hi = last_row / a.n_heads;
    const int pos_lo = a.tok_pos[first_tok + tok_lo], pos_hi = a.tok_pos[first_tok + tok_hi];
    const int key_lo = (a.window > 0 && pos_lo - a.window + 1 > 0) ? pos_lo - a.window + 1 : 0;  // first key any row sees
    // this thread's two rows (g and g + 8): their positions, -1 for rows beyond the sequence's last
    int my_pos[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = r0 + mg * 16 + g + 8 * i;
        my_pos[i] = r < n_rows ? a.tok_pos[first_tok + r / a.n_heads] : -1;
    }
    // ---- the pages this block walks
    const int page_first = key_lo / PAGE, page_last = pos_hi / PAGE;
    const int n_pages_all = page_last - page_first + 1;
    const int per_split = (n_pages_all + a.splits - 1) / a.splits;
    const int my_first = page_first + split * per_split;
    const int my_last = min(my_first + per_split - 1, page_last);
    const int* table = a.block_table + (size_t)a.slots[seq] * a.max_pages;
    const int pieces = width / 8;  // 16-byte pieces of a row

    // a thread's pieces of a page lie THREADS apart: row and piece of the first, and what one step adds (no division in the loop)
    const int lp_row0 = tid / pieces, lp_piece0 = tid - lp_row0 * pieces;
    const int lp_row_step = THREADS / pieces, lp_piece_step = THREADS - lp_row_step * pieces;
    auto load_page = [&](int stage, int page_index) {
        const int page = table[page_index];
        const __nv_bfloat16* src = a.pages + (size_t)page * PAGE * width;
        __nv_bfloat16* dst = k_s + (size_t)stage * PAGE * stride;
        const int row_lo = key_lo - page_index * PAGE, row_hi = pos_hi - page_index * PAGE;  // rows of the page inside the key range
        int row = lp_row0, piece = lp_piece0;
        while (row < PAGE) {
            cp_async_16(dst + row * stride + piece * 8, src + row * width + piece * 8, row >= row_lo && row <= row_hi);
            row += lp_row_step;
            piece += lp_piece_step;
            if (piece >= pieces) {
                piece -= pieces;
                ++row;
            }
        }
    };
    if (my_first <= my_last) load_page(0, my_first);
    cp_async_commit();

    // ---- stage the query tile: the carried part as it is (asynchronous 16-byte copies, zeros for rows beyond the
    // sequence's last), the own part rotated
    {
        const int q_pieces = a.rank / 8;
        for (int i = tid; i < ROWS * q_pieces; i += THREADS) {
            const int r = i / q_pieces, piece = i - r * q_pieces;
            const int row = r0 + r;
            const bool valid = row < n_rows;
            const int t = first_tok + (valid ? row / a.n_heads : 0), h = valid ? row % a.n_heads : 0;
            cp_async_16(q_s + (size_t)r * stride + piece * 8, a.q_carried + (size_t)t * a.qc_tok + (size_t)h * a.qc_head + piece * 8, valid);
        }
        cp_async_commit();
        const int half = a.rot_dims >> 1;
#pragma unroll 4
        for (int i = tid; i < ROWS * a.rot; i += THREADS) {
            const int r = i / a.rot, e = i - r * a.rot;
            const int row = r0 + r;
            float v = 0.f;
            if (row < n_rows) {
                const int t = first_tok + row / a.n_heads, h = row % a.n_heads;
                const __nv_bfloat16* own = a.q_raw + ((size_t)t * a.n_heads + h) * a.q_raw_dim + a.q_rot_at;
                v = __bfloat162float(own[e]);
                if (e < a.rot_dims) {
                    const int f = e < half ? e : e - half;
                    const int pos = a.tok_pos[t];
                    const float c = a.cos_table[(size_t)pos * half + f], sn = a.sin_table[(size_t)pos * half + f];
                    const float other = __bfloat162float(own[e < half ? e + half : e - half]);
                    v = e < half ? v * c - other * sn : v * c + other * sn;
                }
            }
            q_s[(size_t)r * stride + a.rank + e] = __float2bfloat16_rn(v);
        }
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int nt_used = a.rank / 32;          // this warp's 8-column tiles (even: rank is a multiple of 64)
    const int col0 = cg * (a.rank / 4);       // its first output column
    const float sl2 = a.scale * LOG2E;
    const int k_steps = width / 16;

    for (int pi = my_first, it = 0; pi <= my_last; ++pi, ++it) {
        const int stage = it & 1;
        cp_async_wait<0>();
        __syncthreads();  // the page (at the first turn also the query tile) is in shared memory, and every warp is done with the
                          // other stage, the P tile and the statistics of the turn before
        if (pi + 1 <= my_last) load_page(stage ^ 1, pi + 1);  // arrives under this turn's arithmetic
        cp_async_commit();
        const __nv_bfloat16* kt = k_s + (size_t)stage * PAGE * stride;
        // ---- scores of this warp's 16 keys
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
        {
            // 32-bit shared-memory addresses, advanced by 32 bytes a step (no conversion of a generic pointer per ldmatrix)
            const uint32_t q_at = smem_u32(q_s + (size_t)(mg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * stride + (lane >> 4) * 8);
            const uint32_t k_at = smem_u32(kt + (size_t)(cg * 16 + (lane & 7) + (lane >> 4) * 8) * stride + ((lane >> 3) & 1) * 8);
            if constexpr (NT <= 8) {
                // the fragments of the next step are asked for before the products of this one are issued (measured: 4% off
                // the kernel at a latent of 256; at 512, where the accumulator leaves few registers, 7% slower, so not there)
                uint32_t qa0[4], kb0[4], qa1[4], kb1[4];
                ldmatrix_x4_at(qa0, q_at);
                ldmatrix_x4_at(kb0, k_at);
                int ks = 0;
                for (; ks + 2 <= k_steps; ks += 2) {
                    ldmatrix_x4_at(qa1, q_at + (ks + 1) * 32);
                    ldmatrix_x4_at(kb1, k_at + (ks + 1) * 32);
                    mma_16816(s[0], qa0, kb0[0], kb0[1]);
                    mma_16816(s[1], qa0, kb0[2], kb0[3]);
                    if (ks + 2 < k_steps) {
                        ldmatrix_x4_at(qa0, q_at + (ks + 2) * 32);
                        ldmatrix_x4_at(kb0, k_at + (ks + 2) * 32);
                    }
                    mma_16816(s[0], qa1, kb1[0], kb1[1]);
                    mma_16816(s[1], qa1, kb1[2], kb1[3]);
                }
                if (ks < k_steps) {  // an odd number of steps: the last one's fragments are in hand
                    mma_16816(s[0], qa0, kb0[0], kb0[1]);
                    mma_16816(s[1], qa0, kb0[2], kb0[3]);
                }
            } else {
                for (int ks = 0; ks < k_steps; ++ks) {
                    uint32_t qa[4], kb[4];
                    ldmatrix_x4_at(qa, q_at + ks * 32);
                    ldmatrix_x4_at(kb, k_at + ks * 32);
                    mma_16816(s[0], qa, kb[0], kb[1]);
                    mma_16816(s[1], qa, kb[2], kb[3]);
                }
            }
        }
        // ---- mask, and this warp's row maxima
        const int j_base = pi * PAGE + cg * 16;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = c >> 1;  // row g (c = 0, 1) or g + 8 (c = 2, 3)
                const int j = j_base + n * 8 + 2 * tg + (c & 1);
                const bool seen = j <= my_pos[i] && (a.window == 0 || my_pos[i] - j < a.window);
                s[n][c] = seen ? s[n][c] * sl2 : -INFINITY;
                mx[i] = fmaxf(mx[i], s[n][c]);
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        }
        float* smax = stat_max + (stage * MG + mg) * COL_WARPS * 16;  // [stage][tile][quarter][row]
        float* ssum = stat_sum + (stage * MG + mg) * COL_WARPS * 16;
        if (tg == 0) {
            smax[cg * 16 + g] = mx[0];
            smax[cg * 16 + g + 8] = mx[1];
        }
        __syncthreads();
        // ---- the rows' new maxima, probabilities, partial sums; rescale the accumulator
        float corr[2], m_new[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = g + 8 * i;
            float m = m_run[i];
#pragma unroll
            for (int w = 0; w < COL_WARPS; ++w) m = fmaxf(m, smax[w * 16 + r]);
            m_new[i] = m;
            corr[i] = m == -INFINITY ? 1.f : exp2f(m_run[i] - m);
            m_run[i] = m;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            float p[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = c >> 1;
                p[c] = m_new[i] == -INFINITY ? 0.f : exp2f(s[n][c] - m_new[i]);
                sum[i] += p[c];
            }
            const int col = cg * 16 + n * 8 + 2 * tg;
            *reinterpret_cast<uint32_t*>(p_s + (size_t)(mg * 16 + g) * P_STRIDE + col) = pack_bf16(p[0], p[1]);
            *reinterpret_cast<uint32_t*>(p_s + (size_t)(mg * 16 + g + 8) * P_STRIDE + col) = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
            sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
        }
        if (tg == 0) {
            ssum[cg * 16 + g] = sum[0];
            ssum[cg * 16 + g + 8] = sum[1];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n)
            if (n < nt_used) {
                o[n][0] *= corr[0]; o[n][1] *= corr[0];
                o[n][2] *= corr[1]; o[n][3] *= corr[1];
            }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = g + 8 * i;
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < COL_WARPS; ++w) t += ssum[w * 16 + r];
            l_run[i] = l_run[i] * corr[i] + t;
        }
        // ---- output: P [16 x 64] times this warp's columns of V
        {
            const uint32_t p_at = smem_u32(p_s + (size_t)(mg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * P_STRIDE + (lane >> 4) * 8);
            const uint32_t v_at = smem_u32(kt + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * stride + col0 + (lane >> 4) * 8);
            const uint32_t v_step = 16 * stride * 2;  // bytes from one group of 16 keys to the next
#pragma unroll
            for (int kk = 0; kk < PAGE / 16; ++kk) {
                uint32_t pa[4], vb[2][4];  // after unrolling every index below is a constant
                ldmatrix_x4_at(pa, p_at + kk * 32);
                ldmatrix_x4_trans_at(vb[0], v_at + kk * v_step);
#pragma unroll
                for (int n = 0; n < NT; n += 2)
                    if (n < nt_used) {
                        if (n + 2 < nt_used) ldmatrix_x4_trans_at(vb[((n >> 1) + 1) & 1], v_at + kk * v_step + (n + 2) * 16);
                        mma_16816(o[n], pa, vb[(n >> 1) & 1][0], vb[(n >> 1) & 1][1]);
                        mma_16816(o[n + 1], pa, vb[(n >> 1) & 1][2], vb[(n >> 1) & 1][3]);
                    }
            }
        }
        // the next turn's first barrier stands between these reads of the page and of P and their next writes
    }
    cp_async_wait<0>();

    // ---- results
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = r0 + mg * 16 + g + 8 * i;
        if (row >= n_rows) continue;
        const int t = first_tok + row / a.n_heads, h = row % a.n_heads;
        if (a.splits == 1) {
            const float inv = 1.f / l_run[i];
            __nv_bfloat16* dst = a.out + (size_t)t * a.out_tok + (size_t)h * a.out_head + col0;
#pragma unroll
            for (int n = 0; n < NT; ++n)
                if (n < nt_used)
                    *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * tg) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
        } else {
            const size_t grow = (size_t)split * a.n_rows_total + (size_t)t * a.n_heads + h;
            float* dst = a.part_o + grow * a.rank + col0;
#pragma unroll
            for (int n = 0; n < NT; ++n)
                if (n < nt_used) *reinterpret_cast<float2*>(dst + n * 8 + 2 * tg) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
            if (cg == 0 && tg == 0) {
                a.part_ml[grow * 2] = m_run[i];
                a.part_ml[grow * 2 + 1] = l_run[i];
            }
        }
    }
}

// One thread per (token, head, output column): the splits' partial results in split order.  Every thread forms its
// row's weights itself (the statistics are a few numbers, the same for a whole warp), so that none of its loads waits
// for another.  Maxima are in the exponent-of-two scale of the kernel above.
constexpr int MAX_SPLITS = 16;

__global__ void __launch_bounds__(256) latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                           __nv_bfloat16* __restrict__ out, long long out_tok, long long out_head,
                                                           int n_rows_total, int n_heads, int rank, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_rows_total * rank) return;
    const int row = (int)(idx / rank), d = (int)(idx - (long long)row * rank);
    float ms[MAX_SPLITS], ls[MAX_SPLITS], os[MAX_SPLITS];
    const size_t step = (size_t)n_rows_total * rank;
#pragma unroll
    for (int s = 0; s < MAX_SPLITS; ++s) {
        const bool on = s < splits;
        ms[s] = on ? part_ml[((size_t)s * n_rows_total + row) * 2] : -INFINITY;
        ls[s] = on ? part_ml[((size_t)s * n_rows_total + row) * 2 + 1] : 0.f;
        os[s] = on ? part_o[s * step + idx] : 0.f;  // a split that saw nothing left zeros
    }
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < MAX_SPLITS; ++s) m = fmaxf(m, ms[s]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_SPLITS; ++s) {
        const float w = ms[s] == -INFINITY ? 0.f : exp2f(ms[s] - m);
        l = fmaf(ls[s], w, l);
        acc = fmaf(os[s], w, acc);
    }
    const int t = row / n_heads, h = row % n_heads;
    out[(size_t)t * out_tok + (size_t)h * out_head + d] = __float2bfloat16_rn(acc / l);
}

size_t tiled_smem(int width, int mg) {
    return (size_t)(mg * 16 + 2 * PAGE) * (width + 8) * 2 + (size_t)mg * 16 * P_STRIDE * 2 + 4 * (size_t)mg * COL_WARPS * 16 * 4;
}

template <int NT, int MG>
void launch_tiled(const TiledArgs& a, unsigned tiles16, unsigned n_seqs, int width, cudaStream_t s) {
    static bool prepared = false;
    if (!prepared) {
        cudaFuncSetAttribute(attention_latent_tiled_kernel<NT, MG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        prepared = true;
    }
    gk_launch(attention_latent_tiled_kernel<NT, MG>, dim3((tiles16 + MG - 1) / MG, n_seqs, (unsigned)a.splits), dim3(MG * COL_WARPS * 32),
              tiled_smem(width, MG), s, a);
}

template <int NT>
void launch_tiled_rows(const TiledArgs& a, unsigned tiles16, unsigned n_seqs, int width, cudaStream_t s) {
    // as many 16-row tiles a block as a sequence brings (up to four) and as fit in shared memory beside two pages
    static const int forced = getenv("GTAR_B200_LATENT_ROW_TILES") ? atoi(getenv("GTAR_B200_LATENT_ROW_TILES")) : 0;  // for measurements
    if (forced == 1) { launch_tiled<NT, 1>(a, tiles16, n_seqs, width, s); return; }
    if (forced == 2 && tiled_smem(width, 2) <= 200 * 1024) { launch_tiled<NT, 2>(a, tiles16, n_seqs, width, s); return; }
    if (tiles16 >= 4 && tiled_smem(width, 4) <= 200 * 1024) launch_tiled<NT, 4>(a, tiles16, n_seqs, width, s);
    else if (tiles16 >= 2 && tiled_smem(width, 2) <= 200 * 1024) launch_tiled<NT, 2>(a, tiles16, n_seqs, width, s);
    else launch_tiled<NT, 1>(a, tiles16, n_seqs, width, s);
}

}  // namespace

// Shared memory the kernel needs at least (one 16-row tile a block) for rows of `width` = rank + rot.
GK_EXPORT int gk_attention_latent_tiled_smem(int width) { return (int)tiled_smem(width, 1); }

GK_EXPORT int gk_attention_latent_tiled(const void* q_carried, long long qc_tok, long long qc_head, const void* q_raw,
                                        int q_raw_dim, int q_rot_at, const float* cos_table, const float* sin_table,
                                        const void* pages, void* out, long long out_tok, long long out_head, float* part_o,
                                        float* part_ml, const int* tok_pos, const int* cu_q, const int* slots,
                                        const int* block_table, int n_tokens, int n_seqs, int max_q_len, int n_heads, int rank,
                                        int rot, int rot_dims, int max_pages, int page_size, float scale, int window, int splits,
                                        void* stream) {
    GK_REQUIRE(n_tokens >= 0 && n_seqs > 0 && max_q_len > 0 && n_heads > 0, "attention_latent_tiled: bad sizes");
    GK_REQUIRE(rank > 0 && rank % 64 == 0 && rank <= 512 && rot >= 0 && rot % 16 == 0,
               "attention_latent_tiled: rank %d must be a multiple of 64 up to 512 and rot %d a multiple of 16", rank, rot);
    GK_REQUIRE(rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0, "attention_latent_tiled: bad rotation sizes");
    GK_REQUIRE(q_rot_at >= 0 && q_rot_at + rot <= q_raw_dim, "attention_latent_tiled: the rotated part lies outside the head");
    GK_REQUIRE(page_size == PAGE, "attention_latent_tiled: pages must hold %d positions", PAGE);
    GK_REQUIRE(window >= 0 && splits >= 1 && splits <= MAX_SPLITS, "attention_latent_tiled: bad window, or more than %d splits", MAX_SPLITS);
    GK_REQUIRE(splits == 1 || (part_o && part_ml), "attention_latent_tiled: splits need scratch");
    GK_REQUIRE(((uintptr_t)pages & 15) == 0 && ((uintptr_t)out & 3) == 0 && out_tok % 2 == 0 && out_head % 2 == 0,
               "attention_latent_tiled: misaligned pages or output");
    GK_REQUIRE(((uintptr_t)q_carried & 15) == 0 && qc_tok % 8 == 0 && qc_head % 8 == 0,
               "attention_latent_tiled: the carried queries' rows must start at 16-byte boundaries");
    if (n_tokens == 0) return GK_OK;
    GK_REQUIRE(tiled_smem(rank + rot, 1) <= 200 * 1024, "attention_latent_tiled: rows of %d do not fit in shared memory", rank + rot);
    const long long tiles = ((long long)max_q_len * n_heads + 15) / 16;
    GK_REQUIRE(tiles <= 2147483647LL && n_seqs <= 65535, "attention_latent_tiled: too many tiles or sequences");
    TiledArgs a;
    a.q_carried = (const __nv_bfloat16*)q_carried; a.qc_tok = qc_tok; a.qc_head = qc_head;
    a.q_raw = (const __nv_bfloat16*)q_raw; a.q_raw_dim = q_raw_dim; a.q_rot_at = q_rot_at;
    a.cos_table = cos_table; a.sin_table = sin_table; a.pages = (const __nv_bfloat16*)pages;
    a.out = (__nv_bfloat16*)out; a.out_tok = out_tok; a.out_head = out_head; a.part_o = part_o; a.part_ml = part_ml;
    a.tok_pos = tok_pos; a.cu_q = cu_q; a.slots = slots; a.block_table = block_table;
    a.n_heads = n_heads; a.rank = rank; a.rot = rot; a.rot_dims = rot_dims; a.max_pages = max_pages; a.splits = splits;
    a.n_rows_total = n_tokens * n_heads; a.window = window; a.scale = scale;
    cudaStream_t s = (cudaStream_t)stream;
    const int nt = rank / 32;
    if (nt <= 2) launch_tiled_rows<2>(a, (unsigned)tiles, (unsigned)n_seqs, rank + rot, s);
    else if (nt <= 4) launch_tiled_rows<4>(a, (unsigned)tiles, (unsigned)n_seqs, rank + rot, s);
    else if (nt <= 8) launch_tiled_rows<8>(a, (unsigned)tiles, (unsigned)n_seqs, rank + rot, s);
    else launch_tiled_rows<16>(a, (unsigned)tiles, (unsigned)n_seqs, rank + rot, s);
    GK_CHECK_LAUNCH("attention_latent_tiled");
    if (splits > 1) {
        const int rows = n_tokens * n_heads;
        const long long cells = (long long)rows * rank;
        gk_launch(latent_merge_kernel, dim3((unsigned)((cells + 255) / 256)), dim3(256), 0, s, (const float*)part_o, (const float*)part_ml,
                  (__nv_bfloat16*)out, out_tok, out_head, rows, n_heads, rank, splits);
        GK_CHECK_LAUNCH("latent_merge");
    }
    return GK_OK;
}
