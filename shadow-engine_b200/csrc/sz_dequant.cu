// Test kernels: each weight format's decoder on its own, so the decoders can be compared bit for bit with the CPU
// (the role of the reference's kernels/dequant.cu and the exl3_codebook entry of kernels/exl3.cu).
#include "sz_formats.cuh"

template <int TYPE>
__global__ void sz_dequant_kernel(const u8* __restrict__ src, float* __restrict__ dst, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v;
    if (TYPE == SZ_TYPE_F32) v = ((const float*)src)[i];
    else if (TYPE == SZ_TYPE_F16) v = sz_f16_to_f32(((const u16*)src)[i]);
    else if (TYPE == SZ_TYPE_BF16) v = sz_bf16_to_f32(((const u16*)src)[i]);
    else if (TYPE == SZ_TYPE_Q8_0) v = sz_q8_0_at(src + (i >> 5) * 34, (int)(i & 31));
    else v = sz_iq3_s_at(src + (i >> 8) * 110, (int)(i & 255), c_iq3s_grid);
    dst[i] = v;
}

extern "C" int sz_dequant(int type, uint64_t src, int64_t nbytes, uint64_t dst, int64_t n, uint64_t stream) {
    int64_t be, bb;
    switch (type) {
        case SZ_TYPE_F32: be = 1; bb = 4; break;
        case SZ_TYPE_F16: case SZ_TYPE_BF16: be = 1; bb = 2; break;
        case SZ_TYPE_Q8_0: be = 32; bb = 34; break;
        case SZ_TYPE_IQ3_S: be = 256; bb = 110; break;
        default: return sz_fail(SZ_E_TYPE, "sz_dequant: type %d has no block decoder", type);
    }
    if (nbytes < 0 || nbytes % bb != 0 || n != nbytes / bb * be)
        return sz_fail(SZ_E_ARG, "sz_dequant: %lld bytes of type %d for %lld weights", (long long)nbytes, type, (long long)n);
    if (!src || !dst || (src & 3) || (dst & 3)) return sz_fail(SZ_E_ARG, "sz_dequant: null or misaligned pointer");
    if (n == 0) return SZ_OK;
    const dim3 grid((unsigned)((n + 255) / 256)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    const u8* s = (const u8*)src;
    float* d = (float*)dst;
    switch (type) {
        case SZ_TYPE_F32: sz_dequant_kernel<SZ_TYPE_F32><<<grid, block, 0, st>>>(s, d, n); break;
        case SZ_TYPE_F16: sz_dequant_kernel<SZ_TYPE_F16><<<grid, block, 0, st>>>(s, d, n); break;
        case SZ_TYPE_BF16: sz_dequant_kernel<SZ_TYPE_BF16><<<grid, block, 0, st>>>(s, d, n); break;
        case SZ_TYPE_Q8_0: sz_dequant_kernel<SZ_TYPE_Q8_0><<<grid, block, 0, st>>>(s, d, n); break;
        default: sz_dequant_kernel<SZ_TYPE_IQ3_S><<<grid, block, 0, st>>>(s, d, n); break;
    }
    SZ_CUDA(cudaGetLastError());
    return SZ_OK;
}

__global__ void sz_exl3_codebook_kernel(float* dst) {
    const u32 s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < 65536u) dst[s] = sz_exl3_cb2(s);
}

extern "C" int sz_exl3_codebook(uint64_t dst, uint64_t stream) {
    if (!dst || (dst & 3)) return sz_fail(SZ_E_ARG, "sz_exl3_codebook: null or misaligned pointer");
    sz_exl3_codebook_kernel<<<256, 256, 0, (cudaStream_t)stream>>>((float*)dst);
    SZ_CUDA(cudaGetLastError());
    return SZ_OK;
}

// One warp a tile: lane L decodes positions 8 L .. 8 L + 7 and scatters them to W_hat[in][out].
template <int K>
__global__ void sz_exl3_inner_kernel(const u8* __restrict__ blob, int64_t n_in, int64_t n_out, float* __restrict__ dst) {
    const int64_t tile = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int64_t kt = n_in / 16, nt = n_out / 16;
    if (tile >= kt * nt) return;
    const u32* tr = (const u32*)(blob + 2 * n_in + 2 * n_out + 4) + tile * (8 * K);
    u32 st[8];
    SzExl3Tile<K>::states(tr, lane, st);
    const int64_t k = tile / nt, n = tile % nt;
#pragma unroll
    for (int j = 0; j < 8; j++)
        dst[(k * 16 + sz_exl3_row(lane, j)) * n_out + n * 16 + sz_exl3_col(lane, j)] = sz_exl3_cb2(st[j]);
}

extern "C" int sz_exl3_reconstruct_inner(int bits, uint64_t blob, int64_t n_in, int64_t n_out, uint64_t dst, uint64_t stream) {
    if (bits < 1 || bits > 8) return sz_fail(SZ_E_TYPE, "sz_exl3_reconstruct_inner: K = %d", bits);
    if (n_in <= 0 || n_out <= 0 || n_in % 128 || n_out % 128)
        return sz_fail(SZ_E_ARG, "sz_exl3_reconstruct_inner: %lld x %lld is not whole 128-blocks", (long long)n_in, (long long)n_out);
    if (!blob || !dst || (blob & 3) || (dst & 3)) return sz_fail(SZ_E_ARG, "sz_exl3_reconstruct_inner: null or misaligned pointer");
    const int64_t tiles = (n_in / 16) * (n_out / 16);
    const dim3 grid((unsigned)((tiles + 7) / 8)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    const u8* b = (const u8*)blob;
    float* d = (float*)dst;
    switch (bits) {
        case 1: sz_exl3_inner_kernel<1><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
        case 2: sz_exl3_inner_kernel<2><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
        case 3: sz_exl3_inner_kernel<3><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
        case 4: sz_exl3_inner_kernel<4><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
        case 5: sz_exl3_inner_kernel<5><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
        case 6: sz_exl3_inner_kernel<6><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
        case 7: sz_exl3_inner_kernel<7><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
        default: sz_exl3_inner_kernel<8><<<grid, block, 0, st>>>(b, n_in, n_out, d); break;
    }
    SZ_CUDA(cudaGetLastError());
    return SZ_OK;
}
