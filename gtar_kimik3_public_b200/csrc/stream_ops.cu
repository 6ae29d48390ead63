// Row-wise work on the 32-bit residual stream for layers that norm a branch before AND after it, scale it
// per channel, and mix the results of earlier layers into the stream; a short causal convolution over time with
// a per-sequence state; and the tanh form of GELU.  All arithmetic is 32-bit; only inputs that come out of a
// projection and outputs that go into one may be bfloat16.
//
//   merge:   v   = x + scale * (y / sqrt(mean(y^2) + eps_y)) * w_y          (w_y holds the effective weights)
//            kept[n] = v ;  v = sum_{j <= n} mix[j] * kept[j]               (if a history is given)
//            x_out = v ;  z = (v / sqrt(mean(v^2) + eps_z)) * w_z           (if a next norm is given)
//   conv:    g_t = a_t + sum_j w[:, j] * a_(t - taps + 1 + j), a before the sequence's start = 0, a before the
//            step's start read from the sequence's state (its last taps - 1 inputs)
//   state:   after the step the state holds the sequence's last taps - 1 inputs
//
// One block per row with a fixed block size, so the order of a row's sums depends on nothing but the row.

#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

template <typename TY, typename TZ>
__global__ void __launch_bounds__(ROW_THREADS) branch_merge_kernel(
    const float* x, const TY* __restrict__ y, const float* __restrict__ w_y, const float* __restrict__ scale,
    float eps_y, float* __restrict__ kept, long long kept_stride, int n_kept, const float* __restrict__ mix,
    float* x_out, const float* __restrict__ w_z, float eps_z, TZ* __restrict__ z, int width) {
    extern __shared__ float row[];  // width floats
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t at = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += ROW_THREADS) {
        const float v = to_float(y[at + i]);
        row[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float r = 1.f / sqrtf(ss / (float)width + eps_y);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < width; i += ROW_THREADS) {
        float branch = row[i] * r * w_y[i];
        if (scale != nullptr) branch *= scale[i];
        float v = x[at + i] + branch;
        if (kept != nullptr) {
            kept[(size_t)n_kept * kept_stride + at + i] = v;
            float acc = 0.f;
            for (int j = 0; j < n_kept; ++j) acc = fmaf(mix[j], kept[(size_t)j * kept_stride + at + i], acc);
            v = fmaf(mix[n_kept], v, acc);
        }
        x_out[at + i] = v;
        row[i] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (z == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float r2 = 1.f / sqrtf(ss2 / (float)width + eps_z);
    for (int i = threadIdx.x; i < width; i += ROW_THREADS) z[at + i] = from_float<TZ>(row[i] * r2 * w_z[i]);
}

// One thread per (token, channel).  `a` holds the step's inputs, `state` [n_slots, taps - 1, width] the inputs of
// before: entry k of a sequence's state is its input at position  past - (taps - 1) + k.
// `update` (only where every sequence of the step brings ONE token, so that this thread alone reads and writes its
// sequence's entries for the channel): the state is moved on by the token here and no second kernel is needed.
template <typename TO>
__global__ void causal_conv_kernel(const float* __restrict__ a, const float* __restrict__ w, float* state,
                                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                   const int* __restrict__ cu_q, const int* __restrict__ slots, TO* __restrict__ out,
                                   int n_tokens, int width, int taps, int update) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * width) return;
    const int t = (int)(idx / width), c = (int)(idx - (long long)t * width);
    const int seq = tok_seq[t], pos = tok_pos[t];
    const int first = cu_q[seq];      // the sequence's first row in this step
    const int past = pos - (t - first);
    const float own = a[idx];
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        float v;
        if (back == 0) v = own;
        else if (pos - back < 0) v = 0.f;
        else if (t - back >= first) v = a[idx - (long long)back * width];
        else v = state[((size_t)slots[seq] * (taps - 1) + (pos - back - past + taps - 1)) * width + c];
        acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[idx] = from_float<TO>(own + acc);
    if (update && taps > 1) {
        float* mine = state + (size_t)slots[seq] * (taps - 1) * width + c;
        for (int k = 0; k + 1 < taps - 1; ++k) mine[(size_t)k * width] = mine[(size_t)(k + 1) * width];
        mine[(size_t)(taps - 2) * width] = own;
    }
}

// One thread per (sequence, channel): entry k of the new state is the input at position  new_len - (taps - 1) + k,
// taken from the step's rows or, where the step brought fewer than taps - 1 tokens, from entry k + n of the old
// state (read before entry k is written, k going up).
__global__ void conv_state_kernel(const float* __restrict__ a, float* __restrict__ state, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots, int n_seqs, int width, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_seqs * width) return;
    const int seq = (int)(idx / width), c = (int)(idx - (long long)seq * width);
    const int first = cu_q[seq], n = cu_q[seq + 1] - first;
    const int keep = taps - 1;
    float* mine = state + (size_t)slots[seq] * keep * width + c;
    for (int k = 0; k < keep; ++k) {
        const int row = n - keep + k;  // row of the step that holds this position, if not negative
        float v;
        if (row >= 0) v = a[(size_t)(first + row) * width + c];
        else v = mine[(size_t)(k + n) * width];
        mine[(size_t)k * width] = v;
    }
}

template <typename T>
__global__ void gelu_tanh_kernel(const T* __restrict__ in, T* __restrict__ out, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const float z = to_float(in[idx]);
    const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    out[idx] = from_float<T>(0.5f * z * (1.f + tanhf(inner)));
}

}  // namespace

GK_EXPORT int gk_branch_merge(const float* x, const void* y, int y_dtype, const float* w_y, const float* scale, float eps_y,
                              float* kept, long long kept_stride, int n_kept, const float* mix, float* x_out,
                              const float* w_z, float eps_z, void* z, int z_dtype, int n_rows, int width, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(y_dtype) && GK_VALID_DTYPE(z_dtype), "branch_merge: bad dtype code");
    GK_REQUIRE(n_rows >= 0 && width > 0, "branch_merge: bad sizes rows=%d width=%d", n_rows, width);
    GK_REQUIRE(x && y && w_y && x_out, "branch_merge: the stream, the branch and its norm weights are needed");
    GK_REQUIRE(eps_y > 0.f && (z == nullptr || eps_z > 0.f), "branch_merge: eps must be positive");
    GK_REQUIRE((kept == nullptr) == (mix == nullptr) && n_kept >= 0, "branch_merge: a history needs mixing weights");
    GK_REQUIRE((z == nullptr) == (w_z == nullptr), "branch_merge: a next norm needs weights and an output");
    const size_t smem = (size_t)width * sizeof(float);
    GK_REQUIRE(smem <= 200 * 1024, "branch_merge: rows of %d do not fit in shared memory", width);
    if (n_rows == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(y_dtype, TY, {
        GK_DISPATCH_DTYPE(z_dtype, TZ, {
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(branch_merge_kernel<TY, TZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            gk_launch(branch_merge_kernel<TY, TZ>, dim3(n_rows), dim3(ROW_THREADS), smem, s, x, (const TY*)y, w_y, scale, eps_y,
                      kept, kept_stride, n_kept, mix, x_out, w_z, eps_z, (TZ*)z, width);
        })
    })
    GK_CHECK_LAUNCH("branch_merge");
    return GK_OK;
}

GK_EXPORT int gk_causal_conv(const float* a, const float* w, float* state, const int* tok_pos, const int* tok_seq,
                             const int* cu_q, const int* slots, void* out, int out_dtype, int n_tokens, int width, int taps,
                             int update_single_token_state, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(out_dtype), "causal_conv: bad dtype code");
    GK_REQUIRE(n_tokens >= 0 && width > 0 && taps >= 1, "causal_conv: bad sizes");
    GK_REQUIRE(taps == 1 || state != nullptr, "causal_conv: more than one tap needs a state");
    const long long total = (long long)n_tokens * width;
    if (total == 0) return GK_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "causal_conv: too many elements");
    GK_DISPATCH_DTYPE(out_dtype, TO, {
        gk_launch(causal_conv_kernel<TO>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, a, w, state, tok_pos,
                  tok_seq, cu_q, slots, (TO*)out, n_tokens, width, taps, update_single_token_state);
    })
    GK_CHECK_LAUNCH("causal_conv");
    return GK_OK;
}

GK_EXPORT int gk_conv_state(const float* a, float* state, const int* cu_q, const int* slots, int n_seqs, int width, int taps,
                            void* stream) {
    GK_REQUIRE(n_seqs >= 0 && width > 0 && taps >= 1, "conv_state: bad sizes");
    const long long total = (long long)n_seqs * width;
    if (total == 0 || taps == 1) return GK_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    gk_launch(conv_state_kernel, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, a, state, cu_q, slots, n_seqs,
              width, taps);
    GK_CHECK_LAUNCH("conv_state");
    return GK_OK;
}

GK_EXPORT int gk_gelu_tanh(const void* in, void* out, int dtype, long long total, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "gelu_tanh: bad dtype %d", dtype);
    GK_REQUIRE(total >= 0, "gelu_tanh: bad size");
    if (total == 0) return GK_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "gelu_tanh: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(gelu_tanh_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, (const T*)in, (T*)out,
                  total);
    })
    GK_CHECK_LAUNCH("gelu_tanh");
    return GK_OK;
}
