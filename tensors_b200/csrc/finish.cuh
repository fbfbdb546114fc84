// Fixed-order final reductions shared by the kernels that finish a bias gradient or a loss: the same
// device code whether a reduction runs in a launch of its own or batched with others, so the bits do not
// depend on how a caller schedules it.
#pragma once
#include <cstdint>

namespace tfb {

constexpr int kFinishGroups = 32;

// out[c] = sum over row blocks of partial[b][c] for the 32 columns of column block `col_block`: the calling
// block has 32 x 32 threads; group g (threadIdx.y) adds blocks g, g + 32, ... in ascending order (four loads
// in flight), then the 32 group sums are added in ascending order. `sm` is a [32][33] float array.
__device__ __forceinline__ void colsum_finish_block(const float* __restrict__ partial, long long blocks, long long cols,
                                                    long long ld, float* __restrict__ out, long long col_block,
                                                    float (*sm)[33]) {
    const long long c = col_block * 32 + threadIdx.x;
    float s = 0.f;
    if (c < cols) {
        long long b = threadIdx.y;
        for (; b + 3 * kFinishGroups < blocks; b += 4 * kFinishGroups) {
            const float p0 = partial[b * ld + c], p1 = partial[(b + kFinishGroups) * ld + c];
            const float p2 = partial[(b + 2 * kFinishGroups) * ld + c], p3 = partial[(b + 3 * kFinishGroups) * ld + c];
            s += p0; s += p1; s += p2; s += p3;
        }
        for (; b < blocks; b += kFinishGroups) s += partial[b * ld + c];
    }
    sm[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < cols) {
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < kFinishGroups; ++g) t += sm[g][threadIdx.x];
        out[c] = t;
    }
}

// loss = (-1 * sum_r row_loss[r]) * n_inv with 1024 threads (`tid` = the thread's index among them): strided
// per-thread sums, then a shared-memory tree over `sm` (1024 floats).
__device__ __forceinline__ void loss_finish_block(const float* __restrict__ row_loss, long long rows, float n_inv,
                                                  float* __restrict__ loss_out, int tid, float* sm) {
    float s = 0.f;
    for (long long r = tid; r < rows; r += 1024) s += row_loss[r];
    sm[tid] = s;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) {
        if (tid < o) sm[tid] += sm[tid + o];
        __syncthreads();
    }
    if (tid == 0) *loss_out = (-1.0f * sm[0]) * n_inv;
}

}  // namespace tfb
