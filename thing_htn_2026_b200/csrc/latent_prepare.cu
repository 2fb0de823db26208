// Preparation of attention whose keys and values are read out of one low-rank latent per token.
//
// A token's projected row holds, among others, a latent part of `rank` entries and one shared
// key part of `rot` entries that is to be rotated by the token's position.
//
//   latent_norm      c = latent / sqrt(mean(latent^2) + eps) * w   -> [rows, rank], the operand of
//                    the up-projection that gives every head's unrotated key and its value.
//   latent_assemble  from the row's queries [heads][plain | rot], the up-projection's result
//                    [heads * plain keys | heads * values] and the shared key part: queries with
//                    their last `rot` entries rotated; per head the key [plain | rotated shared
//                    part] and the value, written to the paged cache (keys of plain + rot
//                    entries, values of a size of their own).
//
// The rotation pairs entry 2i with entry 2i + 1 of the rotated part: (a, b) with angle t becomes
// (a cos t - b sin t, b cos t + a sin t); cos and sin come from tables [positions, rot / 2]
// (which may carry a common magnitude).  float32 between the load and the one rounding at the
// store; what is only copied is copied as it is.  One block per row.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128) latent_norm_kernel(T* __restrict__ out, const T* __restrict__ src,
                                                          long long src_stride, const float* __restrict__ gain, float eps,
                                                          int rank) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[33];
    const T* row = src + (size_t)blockIdx.x * src_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        ss += v * v;
    }
    const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
        out[(size_t)blockIdx.x * rank + i] = from_f32<T>(to_f32<T>(row[i]) * r * gain[i]);
}

template <typename T>
__global__ void __launch_bounds__(256) latent_assemble_kernel(
    T* __restrict__ q_out, const T* __restrict__ q_src, long long q_stride, const T* __restrict__ shared_src,
    long long shared_stride, const T* __restrict__ up, const float* __restrict__ cos_tab,
    const float* __restrict__ sin_tab, int table_len, const int* __restrict__ row_slot, const int* __restrict__ row_pos,
    PagedKV kv, int n_heads, int plain, int rot, int value_src, int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    const int pos = row_pos[m];
    const int D = plain + rot, DV = kv.value_dim > 0 ? kv.value_dim : kv.head_dim, half = rot / 2;
    if (pos >= table_len) {
        if (threadIdx.x == 0 && err) atomicOr(err, THN_ERR_POSITION_RANGE);
        return;
    }
    const int page = kv.block_table[(size_t)row_slot[m] * kv.bt_stride + pos / kv.page_size];
    const int in_page = pos % kv.page_size;
    if (page < 0 && threadIdx.x == 0 && err) atomicOr(err, THN_ERR_PAGE_UNMAPPED);
    const float* c_row = cos_tab + (size_t)pos * half;
    const float* s_row = sin_tab + (size_t)pos * half;
    const T* q_row = q_src + (size_t)m * q_stride;
    const T* k_shared = shared_src + (size_t)m * shared_stride;
    const T* up_row = up + (size_t)m * n_heads * (plain + value_src);
    T* cache = (T*)kv.base;

    // queries: the plain part as it is, the rest rotated
    for (int e = threadIdx.x; e < n_heads * plain; e += blockDim.x) {
        const int h = e / plain, d = e - h * plain;
        q_out[((size_t)m * n_heads + h) * D + d] = q_row[h * D + d];
    }
    for (int e = threadIdx.x; e < n_heads * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const float a = to_f32<T>(q_row[h * D + plain + 2 * i]), b = to_f32<T>(q_row[h * D + plain + 2 * i + 1]);
        const float c = c_row[i], s = s_row[i];
        T* dst = q_out + ((size_t)m * n_heads + h) * D + plain + 2 * i;
        dst[0] = from_f32<T>(a * c - b * s);
        dst[1] = from_f32<T>(b * c + a * s);
    }
    if (page < 0) return;
    // keys: every head's plain part from the up-projection, then the shared part, rotated
    for (int e = threadIdx.x; e < n_heads * plain; e += blockDim.x) {
        const int h = e / plain, d = e - h * plain;
        cache[kv_offset_sized(kv, page, 0, h, in_page) + d] = up_row[e];
    }
    for (int e = threadIdx.x; e < n_heads * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const float a = to_f32<T>(k_shared[2 * i]), b = to_f32<T>(k_shared[2 * i + 1]);
        const float c = c_row[i], s = s_row[i];
        T* dst = cache + kv_offset_sized(kv, page, 0, h, in_page) + plain + 2 * i;
        dst[0] = from_f32<T>(a * c - b * s);
        dst[1] = from_f32<T>(b * c + a * s);
    }
    // values: the cache's rows may be wider than the values (padded to the keys' size); the rest is zero
    for (int e = threadIdx.x; e < n_heads * DV; e += blockDim.x) {
        const int h = e / DV, d = e - h * DV;
        cache[kv_offset_sized(kv, page, 1, h, in_page) + d] =
            d < value_src ? up_row[n_heads * plain + h * value_src + d] : from_f32<T>(0.f);
    }
}

}  // namespace

// src: rows of the activation type, `rank` entries each, src_stride elements apart; gain float32
// [rank]; out [rows, rank] of the activation type.
THN_API int thn_latent_norm(void* out, const void* src, long long src_stride, const float* gain, float eps, int rows,
                            int rank, int dtype, cudaStream_t stream) {
    THN_CHECK_ARG(rows >= 0 && rank > 0 && src_stride >= rank && eps > 0.f && gain, "latent_norm: bad arguments");
    if (rows == 0) return THN_OK;
    if (dtype == THN_F32)
        thn_launch(latent_norm_kernel<float>, rows, 128, 0, stream, (float*)out, (const float*)src, src_stride, gain, eps, rank);
    else if (dtype == THN_BF16)
        thn_launch(latent_norm_kernel<__nv_bfloat16>, rows, 128, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)src,
                   src_stride, gain, eps, rank);
    else
        THN_CHECK_ARG(false, "latent_norm: unknown dtype %d", dtype);
    return thn_launch_status("latent_norm");
}

// q_src: [heads][plain + rot] per row, rows q_stride elements apart; shared_src: `rot` entries per
// row, rows shared_stride apart; up [rows, heads * plain + heads * value_src]; q_out
// [rows, heads * (plain + rot)].  The cache entry has `heads` kv heads, keys of plain + rot and
// values of value_dim >= value_src entries (what lies beyond a value is written as zero).
THN_API int thn_latent_assemble(void* q_out, const void* q_src, long long q_stride, const void* shared_src,
                                long long shared_stride, const void* up, const float* cos_tab, const float* sin_tab,
                                int table_len, const int* row_slot, const int* row_pos, void* kv_base,
                                const int* block_table, int bt_stride, int page_size, int n_rows, int n_heads, int plain,
                                int rot, int value_dim, int value_src, int dtype, int* err, cudaStream_t stream) {
    THN_CHECK_ARG(n_rows >= 0 && n_heads > 0 && plain >= 0 && rot >= 0 && rot % 2 == 0 && plain + rot > 0 && value_src > 0 &&
                      value_dim >= value_src && page_size > 0,
                  "latent_assemble: bad sizes");
    THN_CHECK_ARG(rot == 0 || (cos_tab && sin_tab), "latent_assemble: a rotated part needs tables");
    if (n_rows == 0) return THN_OK;
    const int D = plain + rot;
    PagedKV kv{kv_base, block_table, bt_stride, n_heads, page_size, D, value_dim == D ? 0 : value_dim};
    if (rot == 0) table_len = 1 << 30;
    if (dtype == THN_F32)
        thn_launch(latent_assemble_kernel<float>, n_rows, 256, 0, stream, (float*)q_out, (const float*)q_src, q_stride,
                   (const float*)shared_src, shared_stride, (const float*)up, cos_tab, sin_tab, table_len, row_slot, row_pos,
                   kv, n_heads, plain, rot, value_src, err);
    else if (dtype == THN_BF16)
        thn_launch(latent_assemble_kernel<__nv_bfloat16>, n_rows, 256, 0, stream, (__nv_bfloat16*)q_out,
                   (const __nv_bfloat16*)q_src, q_stride, (const __nv_bfloat16*)shared_src, shared_stride,
                   (const __nv_bfloat16*)up, cos_tab, sin_tab, table_len, row_slot, row_pos, kv, n_heads, plain, rot, value_src, err);
    else
        THN_CHECK_ARG(false, "latent_assemble: unknown dtype %d", dtype);
    return thn_launch_status("latent_assemble");
}
