// dense.cu -- matmul_vec for PLAIN weight matrices (F32, BF16) with a batch of activation rows:  C[b, m] = sum_k W[m, k] * x[b, k].
//
//   F32 weights : true 32-bit products and sums (no reduced-precision tensor mode) -- the verification-grade path.
//   BF16 weights: the activation is rounded to bfloat16, products are exact in f32, sums are f32.
//
// Three kernels share that arithmetic and differ only in the order of the f32 sums:
//   b <  DENSE_MIN_B             : one warp per output row (matvec.cu: TF32 / TBF16), weights streamed once with 16-byte loads
//   BF16, b >= 32, k % 64 == 0   : tensor cores -- TMA-staged tiles, tcgen05.mma kind::f16 with bf16 operands, f32 accumulator in TMEM
//                                   (prefill_gemm.cu: the same pipeline the quantised prefill path uses, operand format switched)
//   everything else              : the tiled SIMT kernel below (64 x 64 output tile, 16-deep k slices through shared memory, 4 x 4
//                                   outputs per thread, explicit fmaf)
#include <cuda_bf16.h>

#include "common.cuh"

#define DN_TILE 64
#define DN_K 16
#define DN_THREADS 256

__device__ __forceinline__ float dn_load_w(const float* w, int64_t i) { return w[i]; }
__device__ __forceinline__ float dn_load_w(const uint16_t* w, int64_t i) { return __uint_as_float((unsigned)w[i] << 16); }

// grid: (ceil(m / 64), ceil(b / 64)).  Thread (ty, tx) of a 16 x 16 layout owns batch rows ty*4.. and weight rows tx*4.. of the tile.
template <class WT, bool ROUND_X>
__global__ void __launch_bounds__(DN_THREADS) dense_tile_kernel(const WT* __restrict__ W, const float* __restrict__ X, float* __restrict__ C, int m, int b, int k) {
    __shared__ float sw[DN_K][DN_TILE + 4];       // [kk][weight row]
    __shared__ float sx[DN_K][DN_TILE + 4];       // [kk][batch row]
    const int m0 = blockIdx.x * DN_TILE, b0 = blockIdx.y * DN_TILE;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < k; k0 += DN_K) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread; consecutive threads read consecutive k of one row
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int idx = threadIdx.x + e * DN_THREADS;
            const int r = idx >> 4, kk = idx & 15;
            const bool kin = k0 + kk < k;
            sw[kk][r] = (kin && m0 + r < m) ? dn_load_w(W, (int64_t)(m0 + r) * k + k0 + kk) : 0.0f;
            float xv = (kin && b0 + r < b) ? X[(int64_t)(b0 + r) * k + k0 + kk] : 0.0f;
            if (ROUND_X) xv = __bfloat162float(__float2bfloat16_rn(xv));
            sx[kk][r] = xv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < DN_K; kk++) {
            const float4 wv = *(const float4*)&sw[kk][tx * 4];
            const float4 xv = *(const float4*)&sx[kk][ty * 4];
            const float wr[4] = {wv.x, wv.y, wv.z, wv.w}, xr[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xr[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int bi = b0 + ty * 4 + i;
        if (bi >= b) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int mi = m0 + tx * 4 + j;
            if (mi < m) C[(int64_t)bi * m + mi] = acc[i][j];
        }
    }
}

int cc_launch_prefill_bf16(cc_device* dev, const cc_buf* w, const float* x_f32, float* out, int64_t m, int64_t k, int64_t b);   // prefill_gemm.cu
bool cc_prefill_bf16_supported(int64_t m, int64_t k, int64_t b);

bool cc_dense_supported(int wtype, int64_t b) { return (wtype == CC_F32 || wtype == CC_BF16) && b >= 8; }

int cc_launch_dense(cc_device* dev, const cc_buf* w, const float* x, float* out, int64_t m, int64_t k, int64_t b) {
    if (m == 0 || b == 0) return CC_OK;
    if (w->dtype == CC_BF16 && cc_prefill_bf16_supported(m, k, b) && ((uintptr_t)w->plane[0] & 15) == 0)
        return cc_launch_prefill_bf16(dev, w, x, out, m, k, b);
    dim3 grid((unsigned)((m + DN_TILE - 1) / DN_TILE), (unsigned)((b + DN_TILE - 1) / DN_TILE));
    if (w->dtype == CC_F32) dense_tile_kernel<float, false><<<grid, DN_THREADS, 0, dev->stream>>>((const float*)w->plane[0], x, out, (int)m, (int)b, (int)k);
    else if (w->dtype == CC_BF16) dense_tile_kernel<uint16_t, true><<<grid, DN_THREADS, 0, dev->stream>>>((const uint16_t*)w->plane[0], x, out, (int)m, (int)b, (int)k);
    else return cc_fail(dev, CC_ERR_UNSUPPORTED, "dense matmul: weight type %d", w->dtype);
    CC_LAUNCH_CHECK(dev);
    return CC_OK;
}
