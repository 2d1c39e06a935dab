// Urgent-synapse tables of the persistent kernel's split delivery.
//
// A synapse whose dendritic delay is a multiple of the ring length (0 included:
// the ring index is (front + d) mod D, as in the reference,
// presynapticUpdateStrategySIMT.cc:57-389) arrives in the step that follows the
// spike and has to be delivered before that step's neuron update.  These
// kernels copy exactly those synapses of the SPARSE groups into one compressed
// table (row offsets + packed (target, weight) entries; a few MB, so it stays
// in L2) so that the rest of every row can be delivered off the critical path.
// The table is a private copy: it is rebuilt whenever the arrays it came from
// may have changed.
#pragma once

#include "common.cuh"

namespace b200
{
__device__ __forceinline__ bool urgentDelay(unsigned int d, unsigned int D)
{
    return (d % D) == 0u;
}

// len[row] = urgent synapses of the row.  One warp per row.
__global__ void urgentCountKernel(const b200_synapse_group g, unsigned int *len)
{
    const unsigned int lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    const unsigned int D = g.max_den_delay;
    for(unsigned int row = blockIdx.x * warps + (threadIdx.x >> 5); row < g.num_src; row += gridDim.x * warps) {
        const unsigned int n = min(g.row_length[row], g.row_stride);
        const uint8_t *d = g.d + (unsigned long long)row * g.row_stride;
        unsigned int c = 0;
        for(unsigned int j = lane; j < n; j += 32u) c += urgentDelay(d[j], D) ? 1u : 0u;
        #pragma unroll
        for(int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
        if(lane == 0) len[row] = c;
    }
}

// entries[offsets[row] ...) = the row's urgent synapses in row order, as
// (target index, weight bits).
template<typename IndT>
__global__ void urgentFillKernel(const b200_synapse_group g, const unsigned int *offsets, uint2 *entries)
{
    const unsigned int lane = threadIdx.x & 31u, warps = blockDim.x >> 5;
    const unsigned int D = g.max_den_delay;
    const bool constantWeight = (g.wu_model == B200_WU_STATIC_PULSE_CONSTANT_WEIGHT);
    for(unsigned int row = blockIdx.x * warps + (threadIdx.x >> 5); row < g.num_src; row += gridDim.x * warps) {
        const unsigned int n = min(g.row_length[row], g.row_stride);
        const unsigned long long rowStart = (unsigned long long)row * g.row_stride;
        unsigned int at = offsets[row];
        const unsigned int end = offsets[row + 1];
        for(unsigned int j0 = 0; j0 < n; j0 += 32u) {
            const unsigned int j = j0 + lane;
            const bool take = j < n && urgentDelay(g.d[rowStart + j], D);
            const unsigned int ballot = __ballot_sync(0xFFFFFFFFu, take);
            if(take) {
                const unsigned int pos = at + __popc(ballot & ((1u << lane) - 1u));
                if(pos < end) {
                    const float w = constantWeight ? g.wu_params[0] : g.g[rowStart + j];
                    entries[pos] = make_uint2((unsigned int)static_cast<const IndT*>(g.ind)[rowStart + j], __float_as_uint(w));
                }
            }
            at += __popc(ballot);
        }
    }
}
}   // namespace b200
