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
//                      steps: one kernel); steps of several tokens take the kernel that stages
//                      the tokens in shared memory where the rows' alignment allows it
#include <math.h>

#include <algorithm>

#include "common.cuh"

static int g_mlstm_staged = 1;       // 0: steps of several tokens run the kernel without staging too (measurement)
static int g_mlstm_lanes = 0;        // lanes per column in the staged kernel: 8, 16, 32, or 0: by the step's size

namespace {

constexpr int kLanes = 8;            // lanes per column of S
constexpr int kColumns = 16;         // columns per block
constexpr int kThreads = kLanes * kColumns;

// What the state is carried in between a step's first and last token: float beside bfloat16
// activations; double on the true 32-bit path, where the sums over a long prompt would otherwise
// gather float32 roundings that a cancelling n . q magnifies (the state in memory is float32).
template <typename T> struct Carry { using type = float; };
template <> struct Carry<float> { using type = double; };

// Two adjacent entries at once (the address is a multiple of their joint size).
template <typename T> __device__ __forceinline__ float2 load_pair(const T* p);
template <> __device__ __forceinline__ float2 load_pair<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

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
    using A = typename Carry<T>::type;
    A s[R], n[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + kLanes * r;
        s[r] = active && d < D ? (A)s_col[d] : (A)0;
        n[r] = d < D ? (A)nm_block[d] : (A)0;
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
        A top = 0, bottom = 0;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + kLanes * r;
            const float k = d < D ? to_f32<T>(k_src[d]) : 0.f;
            const float q = d < D ? to_f32<T>(q_src[d]) * q_scale : 0.f;
            const A tk = (A)take * k;
            s[r] = (A)keep * s[r] + tk * v;
            n[r] = (A)keep * n[r] + tk;
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
            o[((size_t)row * n_heads + head) * E + column] = (float)(top / (fmax(fabs(bottom), (A)expf(-m)) + (A)floor_));
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + kLanes * r;
        if (d < D) {
            if (active) s_col[d] = (float)s[r];
            if (group == 0) nm_block[d] = (float)n[r];
        }
    }
    if (threadIdx.x == 0) nm_block[D] = m;
}

// The same recurrence for steps of several tokens per sequence, with the tokens' operands staged
// in shared memory: up to kStage tokens at a time (fewer for large keys), the next stage's q, k, v
// and gates copied by cp.async while this stage is worked on.  The running maxima of a stage are
// a short serial chain of additions and comparisons, which every thread walks; the three
// exponentials of a token are then computed by one thread each.  Inside a stage a token costs a
// column's lanes their multiply-adds, three shuffles per sum and one division.  The arithmetic,
// and its order, are those of the kernel above.  Needs rows whose q, k and v parts start on
// 16-byte boundaries (the launcher checks).  A lane takes pairs of adjacent
// entries (one 4-byte load for two bfloat16), and q's scale multiplies the two sums, not every
// entry.  LANES lanes hold a column: 8; 16 and 32 are built for measurement (one prompt of 2,048
// tokens, 16 heads of 128 x 128: 0.80 ms at 8 lanes, 0.80 at 16, 0.89 at 32; 32 heads: 0.98, 1.07,
// 1.46; eight prompts of 16 heads: 2.6, 3.2, 4.8: more lanes give more warps and more instructions
// for the same sums, and no shorter chain per token).
constexpr int kStage = 16;

__device__ __forceinline__ void copy16_async(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void copy4_async(void* smem, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void copy_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

template <typename T, int R, int LANES, bool EXACT>
__global__ void __launch_bounds__(LANES * kColumns) mlstm_recurrence_staged_kernel(
    float* __restrict__ o, float* __restrict__ S, float* __restrict__ nm, const T* __restrict__ proj, int proj_width,
    const float* __restrict__ gates, const int* __restrict__ cu_seqlens, const int* __restrict__ slots, int n_heads, int D,
    int E, float q_scale, float floor_, int stage_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char staged_raw[];
    constexpr int kPer16 = 16 / (int)sizeof(T);                  // elements per 16-byte copy
    const int row_elems = 2 * D + kColumns;                      // q, k, the block's 16 columns of v
    T* buffers = reinterpret_cast<T*>(staged_raw);               // [2][stage_tokens][row_elems]
    float* gate_i = reinterpret_cast<float*>(buffers + (size_t)2 * stage_tokens * row_elems);   // [2][kStage]
    float* gate_f = gate_i + 2 * kStage;                         // [2][kStage]
    float* keep_s = gate_f + 2 * kStage;                         // [kStage] exp(f + m - m')
    float* take_s = keep_s + kStage;                             // [kStage] exp(i - m')
    float* low_s = take_s + kStage;                              // [kStage] exp(-m')
    const int seq = blockIdx.x, head = blockIdx.y, block_of_columns = blockIdx.z;
    constexpr int kBlock = LANES * kColumns;
    const int group = threadIdx.x / LANES, lane = threadIdx.x % LANES;
    const int column = block_of_columns * kColumns + group;
    const bool active = column < E;
    const int slot = slots[seq];
    const int row0 = cu_seqlens[seq], row1 = cu_seqlens[seq + 1];

    float* s_col = S + (((size_t)slot * n_heads + head) * E + (active ? column : 0)) * D;
    float* nm_block = nm + (((size_t)slot * n_heads + head) * gridDim.z + block_of_columns) * (D + 1);
    using A = typename Carry<T>::type;
    // a lane holds the entries 2 lane + 2 LANES j and the one after it, j = 0 .. R / 2 - 1 (D is even here)
    static_assert(R % 2 == 0, "pairs of entries");
    A s[R], n[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = 2 * lane + 2 * LANES * (r >> 1) + (r & 1);
        s[r] = active && d < D ? (A)s_col[d] : (A)0;
        n[r] = d < D ? (A)nm_block[d] : (A)0;
    }
    float m = nm_block[D];

    const int copies_per_row = row_elems / kPer16;
    auto issue = [&](int first_row, int buffer) {
        const int count = min(stage_tokens, row1 - first_row);
        T* dst = buffers + (size_t)buffer * stage_tokens * row_elems;
        for (int c = threadIdx.x; c < count * copies_per_row; c += kBlock) {
            const int t = c / copies_per_row, e = (c - t * copies_per_row) * kPer16;
            const T* src = proj + (size_t)(first_row + t) * proj_width;
            const T* from = e < D ? src + (size_t)head * D + e
                          : e < 2 * D ? src + (size_t)(n_heads + head) * D + (e - D)
                                      : src + (size_t)2 * n_heads * D + (size_t)head * E + block_of_columns * kColumns + (e - 2 * D);
            copy16_async(dst + (size_t)t * row_elems + e, from);
        }
        if (threadIdx.x < count) {
            const float* g = gates + (size_t)(first_row + threadIdx.x) * 2 * n_heads;
            copy4_async(gate_i + buffer * kStage + threadIdx.x, g + head);
            copy4_async(gate_f + buffer * kStage + threadIdx.x, g + n_heads + head);
        }
        copy_commit();
    };

    if (row0 < row1) issue(row0, 0);
    int buffer = 0;
    for (int first_row = row0; first_row < row1; first_row += stage_tokens, buffer ^= 1) {
        const int count = min(stage_tokens, row1 - first_row);
        copy_wait_all();
        __syncthreads();                          // this stage has landed; the other buffer is free again
        if (first_row + stage_tokens < row1) issue(first_row + stage_tokens, buffer ^ 1);
        const float* gi = gate_i + buffer * kStage;
        const float* gf = gate_f + buffer * kStage;
        // the stage's running maxima: the same chain in every thread; a thread keeps the one before its own token
        float running = m, before_mine = m;
        for (int t = 0; t < count; ++t) {
            if (t == (int)threadIdx.x) before_mine = running;
            running = fmaxf(gf[t] + running, gi[t]);
        }
        if ((int)threadIdx.x < count) {
            const int t = threadIdx.x;
            const float m_new = fmaxf(gf[t] + before_mine, gi[t]);
            keep_s[t] = expf(gf[t] + before_mine - m_new);
            take_s[t] = expf(gi[t] - m_new);
            low_s[t] = expf(-m_new);
        }
        m = running;
        __syncthreads();
        const T* stage = buffers + (size_t)buffer * stage_tokens * row_elems;
        // (Unrolling this loop by four, so that the sums, shuffles and divisions of neighbouring tokens
        // might overlap, made it slower: 0.97 against 0.85 ms for 2,048 tokens at 8 lanes.)
        for (int t = 0; t < count; ++t) {
            const T* q_src = stage + (size_t)t * row_elems;
            const T* k_src = q_src + D;
            const float v = active ? to_f32<T>(q_src[2 * D + group]) : 0.f;
            const float keep = keep_s[t], take = take_s[t];
            A top = 0, bottom = 0, top1 = 0, bottom1 = 0;
#pragma unroll
            for (int j = 0; j < R / 2; ++j) {
                const int d = 2 * lane + 2 * LANES * j;
                const bool inside = EXACT || d < D;       // EXACT: the lanes' entries are exactly the key's (D = LANES * R)
                const float2 k = inside ? load_pair<T>(k_src + d) : make_float2(0.f, 0.f);
                const float2 q = inside ? load_pair<T>(q_src + d) : make_float2(0.f, 0.f);
                const A tk0 = (A)take * k.x, tk1 = (A)take * k.y;
                s[2 * j] = (A)keep * s[2 * j] + tk0 * v;
                s[2 * j + 1] = (A)keep * s[2 * j + 1] + tk1 * v;
                n[2 * j] = (A)keep * n[2 * j] + tk0;
                n[2 * j + 1] = (A)keep * n[2 * j + 1] + tk1;
                top += s[2 * j] * q.x;
                top1 += s[2 * j + 1] * q.y;
                bottom += n[2 * j] * q.x;
                bottom1 += n[2 * j + 1] * q.y;
            }
            top = (top + top1) * (A)q_scale;          // q's scale, once for the sum
            bottom = (bottom + bottom1) * (A)q_scale;
#pragma unroll
            for (int w = LANES / 2; w > 0; w >>= 1) {
                top += __shfl_xor_sync(0xffffffffu, top, w);
                bottom += __shfl_xor_sync(0xffffffffu, bottom, w);
            }
            if (active && lane == 0)
                o[((size_t)(first_row + t) * n_heads + head) * E + column] =
                    (float)(top / (fmax(fabs(bottom), (A)low_s[t]) + (A)floor_));
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = 2 * lane + 2 * LANES * (r >> 1) + (r & 1);
        if (d < D) {
            if (active) s_col[d] = (float)s[r];
            if (group == 0) nm_block[d] = (float)n[r];
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
    // Steps of several tokens go through shared memory where every 16-byte copy is aligned and stays
    // inside its row: q, k and v parts of whole 16-byte pieces, and room behind a head's last columns.
    const int unit = 16 / (int)sizeof(T);
    const bool staged = !raw_gates && g_mlstm_staged && D % unit == 0 && E % unit == 0 && proj_width % unit == 0 &&
                        ((uintptr_t)proj & 15) == 0 && ((uintptr_t)gates & 3) == 0 &&
                        (E % kColumns == 0 || n_heads * (2 * D + E) + kColumns <= proj_width);
    if (staged) {
        const int row_bytes = (2 * D + kColumns) * (int)sizeof(T);
        const int stage_tokens = std::max(1, std::min(kStage, 32768 / (2 * row_bytes)));
        const size_t smem = (size_t)2 * stage_tokens * row_bytes + 7 * kStage * sizeof(float);
#define THN_MLSTM_STAGED(R, LANES)                                                                                     \
    do {                                                                                                               \
        if (D == LANES * R)                                                                                            \
            thn_launch_ordered(mlstm_recurrence_staged_kernel<T, R, LANES, true>, grid, LANES * kColumns, smem, stream, \
                               o, S, nm, (const T*)proj, proj_width, gates, cu_seqlens, slots, n_heads, D, E, q_scale,  \
                               floor_, stage_tokens);                                                                   \
        else                                                                                                           \
            thn_launch_ordered(mlstm_recurrence_staged_kernel<T, R, LANES, false>, grid, LANES * kColumns, smem, stream, \
                               o, S, nm, (const T*)proj, proj_width, gates, cu_seqlens, slots, n_heads, D, E, q_scale,  \
                               floor_, stage_tokens);                                                                   \
    } while (0)
        int lanes = g_mlstm_lanes;
        if (lanes == 0) lanes = 8;
        if (lanes == 32) {
            const int per32 = (D + 31) / 32;
            if (per32 <= 2) THN_MLSTM_STAGED(2, 32);
            else if (per32 <= 4) THN_MLSTM_STAGED(4, 32);
            else if (per32 <= 8) THN_MLSTM_STAGED(8, 32);
            else THN_MLSTM_STAGED(16, 32);
        } else if (lanes == 16) {
            const int per16 = (D + 15) / 16;
            if (per16 <= 2) THN_MLSTM_STAGED(2, 16);
            else if (per16 <= 4) THN_MLSTM_STAGED(4, 16);
            else if (per16 <= 8) THN_MLSTM_STAGED(8, 16);
            else if (per16 <= 16) THN_MLSTM_STAGED(16, 16);
            else THN_MLSTM_STAGED(32, 16);
        } else if (per_lane <= 2) THN_MLSTM_STAGED(2, 8);
        else if (per_lane <= 4) THN_MLSTM_STAGED(4, 8);
        else if (per_lane <= 8) THN_MLSTM_STAGED(8, 8);
        else if (per_lane <= 16) THN_MLSTM_STAGED(16, 8);
        else if (per_lane <= 32) THN_MLSTM_STAGED(32, 8);
        else THN_MLSTM_STAGED(64, 8);
#undef THN_MLSTM_STAGED
        return thn_launch_status("mlstm_recurrence");
    }
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

THN_API void thn_set_mlstm_staged(int on, int lanes) {
    g_mlstm_staged = on ? 1 : 0;
    g_mlstm_lanes = lanes == 8 || lanes == 16 || lanes == 32 ? lanes : 0;
}

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
