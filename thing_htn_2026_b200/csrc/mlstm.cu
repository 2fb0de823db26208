// Matrix memory with exponential gating (the mLSTM of xLSTM), as a recurrence over a step's
// tokens from the state that a sequence's earlier steps left.  Per head, with a key size D and
// a value size E, the state is a matrix S [D, E], a vector n [D] and a running maximum m:
//
//     m'  = max(f + m, i)
//     S  <- exp(f + m - m') S + exp(i - m') k v^T        n <- exp(f + m - m') n + exp(i - m') k
//     o   = S^T q / (max(|n . q|, exp(-m')) + floor)
//
// i and f are the logarithms of the input and forget gates: from the pre-activations x, y of a
// head, i = cap tanh((x + b_i) / cap), f = logsigmoid(cap tanh((y + b_f) / cap)).  S, n and m start
// at zero (the cache zeroes a slot's state when it opens).  Everything here is float32; q, k and
// v are read from the projected row in the activation type, q scaled by q_scale in float32.
//
// Every column of S (one entry of v and of o) evolves on its own.  A column is held by 8 lanes
// of a warp, entry d of it by lane d mod 8; n is held the same way by every column's lanes (the
// same arithmetic in the same order everywhere, so all copies are equal), which keeps the
// blocks independent of one another: a block works on one (sequence, head, 16 columns) and
// stores its own copy of n and m, [.., blocks of columns, D + 1] with m last.
//
//   mlstm_gates        x, y -> i, f for every row and head of a step (rows are independent)
//   mlstm_recurrence   the recurrence; with raw_gates it transforms x, y itself (single-token
//                      steps: one kernel)
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kLanes = 8;            // lanes per column of S
constexpr int kColumns = 16;         // columns per block
constexpr int kThreads = kLanes * kColumns;

__device__ __forceinline__ float log_input_gate(float x, float cap) { return cap * tanhf(x / cap); }
__device__ __forceinline__ float log_forget_gate(float y, float cap) {
    const float z = cap * tanhf(y / cap);
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));      // log(logistic(z))
}

__global__ void mlstm_gates_kernel(float* __restrict__ out, const float* __restrict__ pre, const float* __restrict__ bias_i,
                                   const float* __restrict__ bias_f, float cap, long long n, int n_heads) {
    pdl_launch_dependents();
    pdl_wait();
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const int c = (int)(e % (2 * n_heads));
    out[e] = c < n_heads ? log_input_gate(pre[e] + bias_i[c], cap) : log_forget_gate(pre[e] + bias_f[c - n_heads], cap);
}

template <typename T, int R>
__global__ void __launch_bounds__(kThreads) mlstm_recurrence_kernel(
    float* __restrict__ o, float* __restrict__ S, float* __restrict__ nm, const T* __restrict__ proj, int proj_width,
    const float* __restrict__ gates, const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
    int raw_gates, const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int n_heads, int D, int E,
    float q_scale, float floor_) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y, block_of_columns = blockIdx.z;
    const int group = threadIdx.x / kLanes, lane = threadIdx.x % kLanes;
    const int column = block_of_columns * kColumns + group;
    const bool active = column < E;
    const int slot = slots[seq];
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];

    float* s_col = S + (((size_t)slot * n_heads + head) * E + (active ? column : 0)) * D;
    float* nm_block = nm + (((size_t)slot * n_heads + head) * gridDim.z + block_of_columns) * (D + 1);
    float s[R], n[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + kLanes * r;
        s[r] = active && d < D ? s_col[d] : 0.f;
        n[r] = d < D ? nm_block[d] : 0.f;
    }
    float m = nm_block[D];
    const float bi = raw_gates ? bias_i[head] : 0.f, bf = raw_gates ? bias_f[head] : 0.f;

    for (int row = row0; row < row1; ++row) {
        const T* src = proj + (size_t)row * proj_width;
        const T* q_src = src + (size_t)head * D;
        const T* k_src = src + (size_t)(n_heads + head) * D;
        const float v = active ? to_f32<T>(src[(size_t)2 * n_heads * D + (size_t)head * E + column]) : 0.f;
        float gi = gates[(size_t)row * 2 * n_heads + head], gf = gates[(size_t)row * 2 * n_heads + n_heads + head];
        if (raw_gates) {
            gi = log_input_gate(gi + bi, cap);
            gf = log_forget_gate(gf + bf, cap);
        }
        const float m_new = fmaxf(gf + m, gi);
        const float keep = expf(gf + m - m_new), take = expf(gi - m_new);
        float top = 0.f, bottom = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + kLanes * r;
            const float k = d < D ? to_f32<T>(k_src[d]) : 0.f;
            const float q = d < D ? to_f32<T>(q_src[d]) * q_scale : 0.f;
            const float tk = take * k;
            s[r] = keep * s[r] + tk * v;
            n[r] = keep * n[r] + tk;
            top += s[r] * q;
            bottom += n[r] * q;
        }
#pragma unroll
        for (int w = kLanes / 2; w > 0; w >>= 1) {
            top += __shfl_xor_sync(0xffffffffu, top, w);
            bottom += __shfl_xor_sync(0xffffffffu, bottom, w);
        }
        m = m_new;
        if (active && lane == 0)
            o[((size_t)row * n_heads + head) * E + column] = top / (fmaxf(fabsf(bottom), expf(-m)) + floor_);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + kLanes * r;
        if (d < D) {
            if (active) s_col[d] = s[r];
            if (group == 0) nm_block[d] = n[r];
        }
    }
    if (threadIdx.x == 0) nm_block[D] = m;
}

template <typename T>
int launch_recurrence(float* o, float* S, float* nm, const void* proj, int proj_width, const float* gates,
                      const float* bias_i, const float* bias_f, float cap, int raw_gates, const int* cu_seqlens,
                      const int* slots, int n_seqs, int n_heads, int D, int E, float q_scale, float floor_,
                      cudaStream_t stream) {
    const dim3 grid(n_seqs, n_heads, (E + kColumns - 1) / kColumns);
    const int per_lane = (D + kLanes - 1) / kLanes;
#define THN_MLSTM_LAUNCH(R)                                                                                          \
    thn_launch_ordered(mlstm_recurrence_kernel<T, R>, grid, kThreads, 0, stream, o, S, nm, (const T*)proj, proj_width, \
                       gates, bias_i, bias_f, cap, raw_gates, cu_seqlens, slots, n_heads, D, E, q_scale, floor_)
    if (per_lane <= 2) THN_MLSTM_LAUNCH(2);
    else if (per_lane <= 4) THN_MLSTM_LAUNCH(4);
    else if (per_lane <= 8) THN_MLSTM_LAUNCH(8);
    else if (per_lane <= 16) THN_MLSTM_LAUNCH(16);
    else if (per_lane <= 32) THN_MLSTM_LAUNCH(32);
    else THN_MLSTM_LAUNCH(64);
#undef THN_MLSTM_LAUNCH
    return thn_launch_status("mlstm_recurrence");
}

}  // namespace

THN_API int thn_mlstm_columns_per_block() { return kColumns; }

// pre [rows, 2 * heads] (x of every head, then y of every head), biases [heads]; out the same
// shape: i, then f.
THN_API int thn_mlstm_gates(float* out, const float* pre, const float* bias_i, const float* bias_f, float cap, int rows,
                            int n_heads, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && n_heads > 0 && cap > 0.f, "mlstm_gates: bad arguments");
    const long long n = (long long)rows * 2 * n_heads;
    if (n == 0) return THN_OK;
    thn_launch(mlstm_gates_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, out, pre, bias_i, bias_f, cap, n, n_heads);
    return thn_launch_status("mlstm_gates");
}

// proj: rows of the activation type, [q: heads * D | k: heads * D | v: heads * E | ...], proj_width
// elements apart.  gates float32 [rows, 2 * heads]: i and f, or with raw_gates their
// pre-activations (biases and cap are then used).  S float32 [slots, heads, E, D]; nm float32
// [slots, heads, ceil(E / columns per block), D + 1]; o float32 [rows, heads, E].
THN_API int thn_mlstm_recurrence(float* o, float* S, float* nm, const void* proj, int proj_width, const float* gates,
                                 const float* bias_i, const float* bias_f, float cap, int raw_gates,
                                 const int* cu_seqlens, const int* slots, int n_seqs, int n_heads, int key_dim,
                                 int value_dim, float q_scale, float floor_, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(n_seqs >= 0 && n_heads > 0 && key_dim > 0 && value_dim > 0, "mlstm_recurrence: bad sizes");
    THN_CHECK_ARG(proj_width >= n_heads * (2 * key_dim + value_dim), "mlstm_recurrence: rows of %d are too short", proj_width);
    THN_CHECK_ARG(!raw_gates || (bias_i && bias_f && cap > 0.f), "mlstm_recurrence: raw gates need biases and a cap");
    THN_UNSUPPORTED_IF(key_dim > 64 * kLanes, "mlstm_recurrence: key size %d above %d", key_dim, 64 * kLanes);
    THN_UNSUPPORTED_IF(n_heads > 65535 || (value_dim + kColumns - 1) / kColumns > 65535, "mlstm_recurrence: grid too large");
    if (n_seqs == 0) return THN_OK;
    if (dtype == THN_F32)
        return launch_recurrence<float>(o, S, nm, proj, proj_width, gates, bias_i, bias_f, cap, raw_gates, cu_seqlens, slots,
                                        n_seqs, n_heads, key_dim, value_dim, q_scale, floor_, stream);
    if (dtype == THN_BF16)
        return launch_recurrence<__nv_bfloat16>(o, S, nm, proj, proj_width, gates, bias_i, bias_f, cap, raw_gates, cu_seqlens,
                                                slots, n_seqs, n_heads, key_dim, value_dim, q_scale, floor_, stream);
    THN_CHECK_ARG(false, "mlstm_recurrence: unknown dtype %d", dtype);
    return THN_OK;
}
