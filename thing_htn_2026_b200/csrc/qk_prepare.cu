// From a step's projected rows to queries and cache entries, for attention variants that the
// per-head kernel of rope_cache.cu does not cover.  One block per row; everything between
// the load and the one rounding at the store is float32.
//
//   norm scope   0: none.  1: RMS norm per head, gains [head_dim] shared by the heads.
//                2: RMS norm over the whole projection at once (all heads of q, all heads of
//                   k), gains [n_q * head_dim] and [n_kv * head_dim].
//   rotation     the first rotary_dim entries of every head, by the row's position; layout
//                0: entry i is paired with entry i + rotary_dim / 2 (rotate-half);
//                1: entry 2i is paired with entry 2i + 1 (interleaved).
//                The pair (a, b) with angle t becomes (a cos t - b sin t, b cos t + a sin t).
//   values       0: the row brings values of its own, [q | k | v];
//                1: the values are the keys as projected, before norm and rotation, [q | k].
#include "common.cuh"

namespace {
constexpr int kMaxThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kMaxThreads) qk_prepare_kernel(
    T* __restrict__ q_out, const T* __restrict__ proj, int proj_width, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, int norm_scope, float gain_offset, float eps, const float* __restrict__ cos_tab,
    const float* __restrict__ sin_tab, int table_len, int rotary_dim, int interleaved, int values_are_keys,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, PagedKV kv, int n_q, int write_cache,
    int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float vals[];          // [(n_q + n_kv) * D]: q heads, then k heads
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const int D = kv.head_dim;
    const int nq = n_q * D, nk = kv.n_kv * D, total = nq + nk;
    const T* src = proj + (size_t)m * proj_width;
    const int pos = row_pos[m];

    float ss_q = 0.f, ss_k = 0.f;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const float v = to_f32<T>(src[e]);
        vals[e] = v;
        if (e < nq) ss_q += v * v; else ss_k += v * v;
    }
    int page = -1;
    if (write_cache) {
        page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
        if (page < 0) {
            if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
            write_cache = 0;
        }
    }
    const int in_page = pos % kv.page_size;
    // values: untouched copies
    if (write_cache) {
        for (int e = threadIdx.x; e < nk; e += blockDim.x) {
            const int kvh = e / D, d = e - kvh * D;
            const T v = values_are_keys ? src[nq + e] : src[total + e];
            ((T*)kv.base)[kv_offset(kv, page, 1, kvh, in_page) + d] = v;
        }
    }
    if (norm_scope == 2) {
        const float tq = block_sum(ss_q, scratch);
        const float tk = block_sum(ss_k, scratch);
        const float rq = 1.0f / sqrtf(tq / (float)nq + eps), rk = 1.0f / sqrtf(tk / (float)nk + eps);
        for (int e = threadIdx.x; e < total; e += blockDim.x)
            vals[e] = e < nq ? vals[e] * rq * (gain_offset + q_gain[e]) : vals[e] * rk * (gain_offset + k_gain[e - nq]);
    } else if (norm_scope == 1) {
        __syncthreads();
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int head = warp; head < n_q + kv.n_kv; head += blockDim.x >> 5) {
            float ss = 0.f;
            for (int d = lane; d < D; d += 32) ss += vals[head * D + d] * vals[head * D + d];
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)D + eps);
            const float* gain = head < n_q ? q_gain : k_gain;
            for (int d = lane; d < D; d += 32) vals[head * D + d] *= r * (gain_offset + gain[d]);
        }
    }
    __syncthreads();
    const bool rotate = cos_tab != nullptr && rotary_dim > 0;
    if (rotate && pos >= table_len) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        return;
    }
    const int half = rotary_dim / 2;
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const int head = e / D, d = e - head * D;
        float out = vals[e];
        if (rotate && d < rotary_dim) {
            int i, partner;
            bool first;
            if (interleaved) {
                i = d >> 1; first = (d & 1) == 0; partner = e ^ 1;
            } else {
                first = d < half; i = first ? d : d - half; partner = first ? e + half : e - half;
            }
            const float c = cos_tab[(size_t)pos * half + i], s = sin_tab[(size_t)pos * half + i];
            out = first ? out * c - vals[partner] * s : out * c + vals[partner] * s;
        }
        if (e < nq) {
            q_out[(size_t)m * nq + e] = from_f32<T>(out);
        } else if (write_cache) {
            const int kvh = head - n_q;
            ((T*)kv.base)[kv_offset(kv, page, 0, kvh, in_page) + d] = from_f32<T>(out);
        }
    }
}

template <typename T>
int launch(void* q_out, const void* proj, int proj_width, const float* q_gain, const float* k_gain, int norm_scope,
           float gain_offset, float eps, const float* cos_tab, const float* sin_tab, int table_len, int rotary_dim,
           int interleaved, int values_are_keys, const int* row_slot, const int* row_pos, PagedKV kv, int n_rows,
           int n_q, int write_cache, int* err, cudaStream_t stream) {
    const size_t smem = (size_t)(n_q + kv.n_kv) * kv.head_dim * sizeof(float);
    if (smem > 48 * 1024) {
        THN_UNSUPPORTED_IF(smem > 200 * 1024, "qk_prepare: %d heads of %d do not fit shared memory", n_q + kv.n_kv,
                           kv.head_dim);
        cudaFuncSetAttribute(qk_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    const int total = (n_q + kv.n_kv) * kv.head_dim;
    // few rows (single-token steps): the row's latency counts, four values per thread; many rows:
    // 128 threads, more blocks per SM (28.6 against 43.0 us for 2,048 rows of 20 heads of 128)
    int threads = 128;
    if (n_rows <= 64) {
        threads = ((total + 3) / 4 + 31) / 32 * 32;
        threads = threads < 128 ? 128 : threads > kMaxThreads ? kMaxThreads : threads;
    }
    thn_launch(qk_prepare_kernel<T>, n_rows, threads, smem, stream, (T*)q_out, (const T*)proj, proj_width, q_gain,
               k_gain, norm_scope, gain_offset, eps, cos_tab, sin_tab, table_len, rotary_dim, interleaved,
               values_are_keys, row_slot, row_pos, kv, n_q, write_cache, err);
    return thn_launch_status("qk_prepare");
}
}  // namespace

THN_API int thn_qk_prepare(void* q_out, const void* proj, int proj_width, const float* q_gain, const float* k_gain,
                           int norm_scope, float gain_offset, float eps, const float* cos_tab, const float* sin_tab,
                           int table_len, int rotary_dim, int interleaved, int values_are_keys, const int* row_slot,
                           const int* row_pos, void* kv_base, const int* block_table, int bt_stride, int n_kv,
                           int page_size, int head_dim, int n_rows, int n_q, int write_cache, int dtype, int* err,
                           cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_q > 0 && n_kv > 0 && head_dim > 0 && page_size > 0, "qk_prepare: bad sizes");
    THN_CHECK_ARG(norm_scope >= 0 && norm_scope <= 2, "qk_prepare: norm scope %d", norm_scope);
    THN_CHECK_ARG(norm_scope == 0 || (q_gain && k_gain && eps > 0.f), "qk_prepare: a norm needs gains and eps");
    THN_CHECK_ARG(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                  "qk_prepare: rotary_dim %d must be even and within the head size %d", rotary_dim, head_dim);
    THN_CHECK_ARG(proj_width >= (n_q + (values_are_keys ? 1 : 2) * n_kv) * head_dim, "qk_prepare: rows of %d are too short",
                  proj_width);
    if (n_rows == 0) return THN_OK;
    PagedKV kv{kv_base, block_table, bt_stride, n_kv, page_size, head_dim};
    if (dtype == THN_F32)
        return launch<float>(q_out, proj, proj_width, q_gain, k_gain, norm_scope, gain_offset, eps, cos_tab, sin_tab,
                             table_len, rotary_dim, interleaved, values_are_keys, row_slot, row_pos, kv, n_rows, n_q,
                             write_cache, err, stream);
    if (dtype == THN_BF16)
        return launch<__nv_bfloat16>(q_out, proj, proj_width, q_gain, k_gain, norm_scope, gain_offset, eps, cos_tab,
                                     sin_tab, table_len, rotary_dim, interleaved, values_are_keys, row_slot, row_pos, kv,
                                     n_rows, n_q, write_cache, err, stream);
    THN_CHECK_ARG(false, "qk_prepare: unknown dtype %d", dtype);
    return THN_OK;
}
