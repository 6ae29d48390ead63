// The gated delta rule with a decay per head and key channel, as a recurrent mixer: what stands between its
// input projections and its output projection.
//
// Per sequence and head, with a state S [d, dv] of 32-bit floats that starts at zero:
//     S <- diag(g_t) S ;  u_t = beta_t (v_t - S^T k_t) ;  S <- S + k_t u_t^T ;  o_t = S^T q_t
// where q_t, k_t come out of a short causal convolution over time and SiLU and are scaled to unit length per
// head (q also by d^-1/2), v_t out of a convolution and SiLU, beta_t = sigmoid(b_t) and
// g_t = exp(-exp(A_h) * softplus(a_t + dt_bias)) per key channel.  The read-out of a head is divided by its root
// mean square, multiplied by a weight shared by the heads and by sigmoid(gate).
//
// Four kernels:
//   delta_prepare   one warp per token and head: convolutions (the inputs before the step's first token come from the
//                   sequence's state: its last taps - 1 inputs), SiLU, unit lengths, decays and beta, all 32-bit
//   conv_roll       moves every sequence's convolution state on by the step's inputs (steps of one token a sequence: the
//                   prepare kernel does it itself)
//   delta_scan      the recurrence.  A column of S (one value channel) never meets another column, so the work is
//                   cut by (sequence, head, group of columns); a column's d entries are spread over eight adjacent
//                   lanes.  Tokens are staged in shared memory some at a time.  With a = (gS)^T k, b = (gS)^T q and
//                   c = k . q, the token's u = beta (v - a) and o = b + u c: one round of shuffles a token.
//                   One code path serves prompts, portions of prompts and single tokens: the state is read from the
//                   sequence's slot at the start and written back at the end, so a token's result does not depend
//                   on how the sequence was cut.
//   head_norm_gate  one warp per (token, head): RMS norm over the head's values, weight, sigmoid gate
//
// All per-step numbers (starts, slots) are read from device memory.

#include "common.cuh"

namespace {

constexpr int PREP_THREADS = 128;
constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// proj [T, ld]: q (G d) | k (G d) | v (H dv) | b (H) | ...;  low [T, ld_low]: a (H d) | gate (H dv)
// A warp per (token, unit): units 0 .. 2G-1 are the heads of q and of k (convolution, SiLU, unit length), units 2G .. 2G+H-1
// the value heads (convolution and SiLU of the head's values, its decays and its beta).
// `roll`: the step brings this sequence one token, and the thread moves the channel's state on itself (row r takes row
// r + 1, the last row the token's input); only this thread touches the channel, so nothing else can read a row too late.
template <typename T>
__device__ __forceinline__ float conv_silu(const T* __restrict__ proj, long long ld, const float* __restrict__ conv_w,
                                           float* conv_state, size_t slot, int t, int in_step, int c, int C, int taps, bool roll) {
    float y = 0.f;
    for (int j = 0; j < taps; ++j) {  // j tokens back
        const int at = in_step - j;
        float x;
        if (at >= 0) x = to_float(proj[(size_t)(t - j) * ld + c]);
        else x = conv_state[(slot * (taps - 1) + (taps - 1 + at)) * C + c];
        y = fmaf(conv_w[(size_t)c * taps + (taps - 1 - j)], x, y);
    }
    if (roll && taps > 1) {
        float* mine = conv_state + slot * (taps - 1) * C + c;
        for (int r = 0; r + 1 < taps - 1; ++r) mine[(size_t)r * C] = mine[(size_t)(r + 1) * C];
        mine[(size_t)(taps - 2) * C] = to_float(proj[(size_t)t * ld + c]);
    }
    return silu_f(y);
}

constexpr int PREP_PER_LANE = 8;  // a head's channels a lane holds: heads of up to 256

template <typename T, typename TL>
__global__ void __launch_bounds__(PREP_THREADS) delta_prepare_kernel(
    const T* __restrict__ proj, long long ld, const TL* __restrict__ low, long long ld_low,
    const float* __restrict__ conv_w /* [C, taps] */, float* conv_state /* [slots, taps-1, C] */,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ cu_q, const int* __restrict__ slots,
    float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out, float* __restrict__ g_out,
    float* __restrict__ beta_out, int n_tokens, int n_heads, int n_kv, int d, int dv, int taps, int roll_single) {
    pdl_launch_dependents();
    pdl_wait();
    // a warp per (token, unit); a lane's sums run in index order and the lanes meet in warp_sum's fixed order
    const int lane = threadIdx.x & 31, units = 2 * n_kv + n_heads;
    const long long item = (long long)blockIdx.x * (PREP_THREADS / 32) + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * units) return;
    const int t = (int)(item / units), unit = (int)(item - (long long)t * units);
    const int seq = tok_seq[t];
    const int in_step = t - cu_q[seq];
    const size_t slot = (size_t)slots[seq];
    const int qk = n_kv * d, C = 2 * qk + n_heads * dv;
    if (unit < 2 * n_kv) {
        float act[PREP_PER_LANE];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < PREP_PER_LANE; ++e) {
            const int i = lane + 32 * e;
            act[e] = i < d ? conv_silu(proj, ld, conv_w, conv_state, slot, t, in_step, unit * d + i, C, taps, roll_single != 0) : 0.f;
            ss = fmaf(act[e], act[e], ss);
        }
        ss = warp_sum(ss);
        float r = 1.f / sqrtf(ss + 1e-6f);
        const bool is_q = unit < n_kv;
        if (is_q) r *= 1.f / sqrtf((float)d);
        float* dst = (is_q ? q_out : k_out) + ((size_t)t * n_kv + (is_q ? unit : unit - n_kv)) * d;
#pragma unroll
        for (int e = 0; e < PREP_PER_LANE; ++e)
            if (lane + 32 * e < d) dst[lane + 32 * e] = act[e] * r;
        return;
    }
    const int h = unit - 2 * n_kv;
    for (int i = lane; i < dv; i += 32)
        v_out[((size_t)t * n_heads + h) * dv + i] = conv_silu(proj, ld, conv_w, conv_state, slot, t, in_step, 2 * qk + h * dv + i, C, taps, roll_single != 0);
    const float rate = -expf(a_log[h]);
    for (int i = lane; i < d; i += 32) {
        const float step = softplus_f(to_float(low[(size_t)t * ld_low + (size_t)h * d + i]) + dt_bias[h * d + i]);
        g_out[((size_t)t * n_heads + h) * d + i] = expf(rate * step);
    }
    if (lane == 0) beta_out[(size_t)t * n_heads + h] = sigmoid_f(to_float(proj[(size_t)t * ld + C + h]));
}

// state[slot, r, c], r = 0 .. taps-2, oldest first.  After a step of n tokens row r holds the input n - (taps-1) + r of
// the step, or, where that lies before the step, the old row r + n.  A thread walks the rows of its channel upward,
// so every old row is read before it is overwritten.
template <typename T>
__global__ void conv_roll_kernel(const T* __restrict__ proj, long long ld, float* __restrict__ state,
                                 const int* __restrict__ cu_q, const int* __restrict__ slots, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int t0 = cu_q[seq], n = cu_q[seq + 1] - t0;
    float* mine = state + (size_t)slots[seq] * (taps - 1) * C + c;
    for (int r = 0; r < taps - 1; ++r) {
        const int at = n - (taps - 1) + r;
        mine[(size_t)r * C] = at >= 0 ? to_float(proj[(size_t)(t0 + at) * ld + c]) : mine[(size_t)(r + n) * C];
    }
}

constexpr int SCAN_THREADS = 256;  // at most
constexpr int SCAN_COLS = 32;      // at most 32 columns a block (the host launches fewer where the device would stand idle)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// LPC: lanes that share a column of the state; R: state entries a lane holds (d <= LPC * R); TB: tokens staged at a
// time.  A lane's entries are the rows lane * R .. lane * R + R - 1; in shared memory a lane's piece of a vector starts
// at lane * PIECE floats, padded so that the 16-byte loads of the lanes fall into different banks.  A token's step is
// one chain of dependent instructions of a warp (it showed as 209 instructions a token at three cycles each with eight
// lanes a column and sixteen rows a lane): more lanes a column shorten the chain and lengthen the exchange.
template <int R, int TB, int LPC>
__global__ void __launch_bounds__(SCAN_THREADS) delta_scan_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
    const float* __restrict__ beta, float* __restrict__ state /* [slots, H, d, dv] */, float* __restrict__ out /* [T, H, dv] */,
    const int* __restrict__ cu_q, const int* __restrict__ slots, int n_heads, int n_kv, int d, int dv) {
    constexpr int PIECE = R == 4 ? 4 : R + 4, VEC = LPC * PIECE;
    __shared__ __align__(16) float sq[2][TB][VEC], sk[2][TB][VEC], sg[2][TB][VEC];
    __shared__ __align__(16) float sv[2][TB][SCAN_COLS], sb[2][TB];
    pdl_launch_dependents();
    const int n_threads = blockDim.x, n_cols = n_threads / LPC;  // columns of this block
    const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * n_cols;
    const int hk = head / (n_heads / n_kv);
    const int sub = threadIdx.x % LPC, col = col0 + threadIdx.x / LPC;
    const bool live = col < dv;
    // the pieces beyond d stay zero in every stage: those rows of the state never leave zero
    for (int i = threadIdx.x; i < 2 * TB * VEC; i += n_threads) {
        (&sq[0][0][0])[i] = 0.f;
        (&sk[0][0][0])[i] = 0.f;
        (&sg[0][0][0])[i] = 0.f;
    }
    __syncthreads();
    pdl_wait();
    const int t0 = cu_q[seq], n = cu_q[seq + 1] - t0;
    float* my_state = state + (((size_t)slots[seq] * n_heads + head) * d) * dv + col;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = sub * R + r;
        S[r] = (live && row < d) ? my_state[(size_t)row * dv] : 0.f;
    }
    const int quads = d / 4;  // 16-byte pieces of a vector of this head
    auto stage = [&](int buf, int first) {
        const int count = min(TB, n - first);
        if (n_threads % quads == 0) {  // a thread's piece of a vector is the same for every token it copies
            const int c4 = (threadIdx.x % quads) * 4, step = n_threads / quads;
            const int at = (c4 / R) * PIECE + c4 % R;
            const float* pq_ = q + ((size_t)(t0 + first) * n_kv + hk) * d + c4;
            const float* pk_ = k + ((size_t)(t0 + first) * n_kv + hk) * d + c4;
            const float* pg_ = g + ((size_t)(t0 + first) * n_heads + head) * d + c4;
            for (int tt = threadIdx.x / quads; tt < count; tt += step) {
                cp_async16(&sq[buf][tt][at], pq_ + (size_t)tt * n_kv * d);
                cp_async16(&sk[buf][tt][at], pk_ + (size_t)tt * n_kv * d);
                cp_async16(&sg[buf][tt][at], pg_ + (size_t)tt * n_heads * d);
            }
        } else {
            for (int i = threadIdx.x; i < count * quads; i += n_threads) {
                const int tt = i / quads, c4 = (i - tt * quads) * 4;
                const int lane_of = c4 / R, within = c4 - lane_of * R;
                const int at = lane_of * PIECE + within;
                const size_t tok = (size_t)(t0 + first + tt);
                cp_async16(&sq[buf][tt][at], q + (tok * n_kv + hk) * d + c4);
                cp_async16(&sk[buf][tt][at], k + (tok * n_kv + hk) * d + c4);
                cp_async16(&sg[buf][tt][at], g + (tok * n_heads + head) * d + c4);
            }
        }
        for (int i = threadIdx.x; i < count * n_cols; i += n_threads) {
            const int tt = i / n_cols, cc = i - tt * n_cols;
            if (col0 + cc < dv) cp_async4(&sv[buf][tt][cc], v + ((size_t)(t0 + first + tt) * n_heads + head) * dv + col0 + cc);
        }
        if (threadIdx.x < count) cp_async4(&sb[buf][threadIdx.x], beta + (size_t)(t0 + first + threadIdx.x) * n_heads + head);
        cp_async_commit();
    };
    stage(0, 0);
    int buf = 0;
    for (int first = 0; first < n; first += TB, buf ^= 1) {
        if (first + TB < n) {
            stage(buf ^ 1, first + TB);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int count = min(TB, n - first);
        float* out_at = out + ((size_t)(t0 + first) * n_heads + head) * dv + col;
        const float* v_at = &sv[buf][0][threadIdx.x / LPC];
        const float* b_at = &sb[buf][0];
        // every address of the loop moves on by a constant a token
        const float4* pq = reinterpret_cast<const float4*>(&sq[buf][0][sub * PIECE]);
        const float4* pk = reinterpret_cast<const float4*>(&sk[buf][0][sub * PIECE]);
        const float4* pg = reinterpret_cast<const float4*>(&sg[buf][0][sub * PIECE]);
        const size_t out_step = (size_t)n_heads * dv;
#pragma unroll 2
        for (int tt = 0; tt < count; ++tt, out_at += out_step, v_at += SCAN_COLS, ++b_at, pq += VEC / 4, pk += VEC / 4, pg += VEC / 4) {
            float kk[R], qq[R];
            // four partial sums each (one per place in a group of four rows): chains of R / 4 dependent operations
            float a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f}, c4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r4 = 0; r4 < R / 4; ++r4) {
                const float4 g4 = pg[r4], k4 = pk[r4], q4 = pq[r4];
                const float gs[4] = {g4.x, g4.y, g4.z, g4.w};
                kk[4 * r4] = k4.x; kk[4 * r4 + 1] = k4.y; kk[4 * r4 + 2] = k4.z; kk[4 * r4 + 3] = k4.w;
                qq[4 * r4] = q4.x; qq[4 * r4 + 1] = q4.y; qq[4 * r4 + 2] = q4.z; qq[4 * r4 + 3] = q4.w;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = 4 * r4 + e;
                    S[r] *= gs[e];
                    a4[e] = fmaf(S[r], kk[r], a4[e]);
                    b4[e] = fmaf(S[r], qq[r], b4[e]);
                    c4[e] = fmaf(kk[r], qq[r], c4[e]);
                }
            }
            float a = (a4[0] + a4[1]) + (a4[2] + a4[3]), b = (b4[0] + b4[1]) + (b4[2] + b4[3]), c = (c4[0] + c4[1]) + (c4[2] + c4[3]);
#pragma unroll
            for (int o = 1; o < LPC; o <<= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                b += __shfl_xor_sync(0xffffffffu, b, o);
                c += __shfl_xor_sync(0xffffffffu, c, o);
            }
            const float u = *b_at * (*v_at - a);
#pragma unroll
            for (int r = 0; r < R; ++r) S[r] = fmaf(kk[r], u, S[r]);
            if (live && sub == 0) *out_at = fmaf(u, c, b);
        }
        __syncthreads();  // the stage is free for the load after next
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = sub * R + r;
        if (live && row < d) my_state[(size_t)row * dv] = S[r];
    }
}

template <typename T, typename TL>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, const TL* __restrict__ gate,
                                      long long ld_gate, T* __restrict__ out, long long n_rows, int n_heads, int dv, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = row / n_heads;
    const int h = (int)(row - t * n_heads);
    const float* x = o + (size_t)row * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)dv + eps);
    const TL* gt = gate + (size_t)t * ld_gate + (size_t)h * dv;
    for (int i = lane; i < dv; i += 32) out[(size_t)row * dv + i] = from_float<T>(x[i] * r * weight[i] * sigmoid_f(to_float(gt[i])));
}

}  // namespace

GK_EXPORT int gk_delta_prepare(const void* proj, int dtype, long long ld, const void* low, int low_dtype, long long ld_low,
                               const float* conv_w, float* conv_state, const float* a_log, const float* dt_bias,
                               const int* tok_pos, const int* tok_seq, const int* cu_q, const int* slots, float* q_out,
                               float* k_out, float* v_out, float* g_out, float* beta_out, int n_tokens, int n_heads, int n_kv,
                               int d, int dv, int taps, int roll_single, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && GK_VALID_DTYPE(low_dtype), "delta_prepare: bad dtype");
    GK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0 && d > 0 && dv > 0, "delta_prepare: bad sizes");
    GK_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "delta_prepare: %d taps (1 to %d)", taps, MAX_TAPS);
    GK_REQUIRE(taps == 1 || conv_state != nullptr, "delta_prepare: a convolution of several taps needs its state");
    if (n_tokens == 0) return GK_OK;
    GK_REQUIRE(d <= 32 * PREP_PER_LANE, "delta_prepare: key heads of %d are more than a warp holds (%d)", d, 32 * PREP_PER_LANE);
    const long long items = (long long)n_tokens * (2 * n_kv + n_heads);
    const long long blocks = (items + PREP_THREADS / 32 - 1) / (PREP_THREADS / 32);
    GK_REQUIRE(blocks < 2147483647LL, "delta_prepare: too many tokens");
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(dtype, T, {
        GK_DISPATCH_DTYPE(low_dtype, TL, {
            gk_launch(delta_prepare_kernel<T, TL>, dim3((unsigned)blocks), dim3(PREP_THREADS), 0, s, (const T*)proj, ld, (const TL*)low,
                      ld_low, conv_w, conv_state, a_log, dt_bias, tok_pos, tok_seq, cu_q, slots, q_out, k_out, v_out, g_out,
                      beta_out, n_tokens, n_heads, n_kv, d, dv, taps, roll_single);
        })
    })
    GK_CHECK_LAUNCH("delta_prepare");
    return GK_OK;
}

GK_EXPORT int gk_conv_roll(const void* proj, int dtype, long long ld, float* state, const int* cu_q, const int* slots,
                           int n_seqs, int channels, int taps, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "conv_roll: bad dtype %d", dtype);
    GK_REQUIRE(taps >= 1 && taps <= MAX_TAPS && channels > 0, "conv_roll: bad sizes");
    if (n_seqs == 0 || taps == 1) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(conv_roll_kernel<T>, dim3((channels + 255) / 256, n_seqs), dim3(256), 0, s, (const T*)proj, ld, state, cu_q,
                  slots, channels, taps);
    })
    GK_CHECK_LAUNCH("conv_roll");
    return GK_OK;
}

GK_EXPORT int gk_delta_scan(const float* q, const float* k, const float* v, const float* g, const float* beta, float* state,
                            float* out, const int* cu_q, const int* slots, int n_seqs, int n_heads, int n_kv, int d, int dv,
                            int lanes, int force_cols, void* stream) {
    GK_REQUIRE(n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "delta_scan: bad head counts %d/%d", n_heads, n_kv);
    GK_REQUIRE(d > 0 && d % 4 == 0 && d <= 256, "delta_scan: key size %d must be a multiple of 4, at most 256", d);
    GK_REQUIRE(dv > 0 && n_seqs >= 0 && n_seqs <= 65535 && n_heads <= 65535, "delta_scan: bad sizes");
    if (n_seqs == 0) return GK_OK;
    // Few (sequence, head) pairs: fewer columns a block, so that the columns of a head spread over more SMs and a token's
    // step is not held up by the block's other warps asking shared memory for the same vectors.
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    // The choice goes by the key size alone (the lanes' sums meet in another order with another number of lanes, and a
    // token's result must not depend on what else is in the step).  Measured on 2,048 tokens of one sequence, 8 / 16 / 32
    // lanes: heads of 64: 470 / 438 / 432 us; of 128: 664 / 600 / 607 (8 heads), 688 / 713 / 813 (16 heads), and 8 lanes
    // are the fastest with many sequences (64 single tokens: 79 / 116 / 196 us); of 256: 1,407 / 900 / 1,031.
    if (lanes == 0) lanes = d <= 32 ? 8 : d <= 64 ? 16 : d <= 128 ? 8 : 16;
    GK_REQUIRE(lanes == 8 || lanes == 16 || lanes == 32, "delta_scan: 8, 16 or 32 lanes a column, not %d", lanes);
    if (d <= 32) lanes = 8;
    else if (d <= 64 && lanes == 32) lanes = 16;
    int cols = SCAN_THREADS / lanes;
    while (cols > 2 && cols * lanes > 64 && (long long)n_seqs * n_heads * ((dv + cols - 1) / cols) < 2LL * sms) cols /= 2;
    if (force_cols > 0 && force_cols * lanes <= SCAN_THREADS && force_cols <= SCAN_COLS) cols = force_cols;
    const dim3 grid((dv + cols - 1) / cols, n_heads, n_seqs), block(cols * lanes);
    cudaStream_t s = (cudaStream_t)stream;
#define GK_SCAN(R, TB, L)                                                                                                \
    gk_launch(delta_scan_kernel<R, TB, L>, grid, block, 0, s, q, k, v, g, beta, state, out, cu_q, slots, n_heads, n_kv, d, dv)
    if (lanes == 8) {
        if (d <= 32) GK_SCAN(4, 16, 8);
        else if (d <= 64) GK_SCAN(8, 16, 8);
        else if (d <= 128) GK_SCAN(16, 8, 8);
        else GK_SCAN(32, 4, 8);
    } else if (lanes == 16) {
        if (d <= 64) GK_SCAN(4, 16, 16);
        else if (d <= 128) GK_SCAN(8, 8, 16);
        else GK_SCAN(16, 4, 16);
    } else {
        if (d <= 128) GK_SCAN(4, 8, 32);
        else GK_SCAN(8, 4, 32);
    }
#undef GK_SCAN
    GK_CHECK_LAUNCH("delta_scan");
    return GK_OK;
}

GK_EXPORT int gk_head_norm_gate(const float* o, const float* weight, const void* gate, int gate_dtype, long long ld_gate,
                                void* out, int out_dtype, long long n_tokens, int n_heads, int dv, float eps, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(gate_dtype) && GK_VALID_DTYPE(out_dtype), "head_norm_gate: bad dtype");
    GK_REQUIRE(n_heads > 0 && dv > 0, "head_norm_gate: bad sizes");
    if (n_tokens == 0) return GK_OK;
    const long long rows = n_tokens * n_heads;
    const long long blocks = (rows + 7) / 8;
    GK_REQUIRE(blocks < 2147483647LL, "head_norm_gate: too many rows");
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(out_dtype, T, {
        GK_DISPATCH_DTYPE(gate_dtype, TL, {
            gk_launch(head_norm_gate_kernel<T, TL>, dim3((unsigned)blocks), dim3(256), 0, s, o, weight, (const TL*)gate, ld_gate,
                      (T*)out, rows, n_heads, dv, eps);
        })
    })
    GK_CHECK_LAUNCH("head_norm_gate");
    return GK_OK;
}
