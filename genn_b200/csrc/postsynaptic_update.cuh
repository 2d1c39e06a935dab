// Postsynaptic (learning) update and batch-reduce custom update kernels.
//
// postsynapticUpdateKernel replaces updatePostsynapticKernel
// (backendSIMT.cc:766-803, 1822-1898): for every spike of the TARGET population
// walk that neuron's column through the column-major remap and run the
// post-spike half of the learning rule (STDP potentiation,
// weightUpdateModels.h:362-368).  Work item = (post spike, 128-entry tile of
// its column); the remap read is coalesced, the weight read-modify-write is a
// gather/scatter over the row-major weight array (12 algorithmic bytes per
// event: 4 remap + 4 weight read + 4 weight write).
//
// batchReduceKernel replaces the batch branch of the custom-update kernels
// (backendSIMT.cc:888-927, 1109-1147): one thread per element walks the batch
// dimension (stride E, so every step is a coalesced line per warp), keeps the
// running sum or maximum in a register and writes the reduced value once;
// optionally it scales and broadcasts the result back into every batch copy.
#pragma once

#include "common.cuh"
#include "presynaptic_update.cuh"

namespace b200
{
constexpr int POST_BLOCK = 128;

__global__ void __launch_bounds__(POST_BLOCK)
postsynapticUpdateKernel(const SynapseLaunch L)
{
    const unsigned int gi = findGroup(L.block_start, L.num_groups, blockIdx.x);
    const b200_synapse_group &g = L.groups[gi];
    const unsigned int tile = blockIdx.x - __ldg(&L.block_start[gi]);
    const unsigned int b = blockIdx.z;
    const unsigned int k = L.state->phase;
    const unsigned int tslots = g.trg_delay_slots;
    const unsigned int rslot = ringSlot(k + tslots - g.back_prop_delay, tslots);
    const unsigned int count = g.trg_spk_cnt[b * tslots + rslot];
    if(blockIdx.y >= count) return;
    const unsigned int *spk = g.trg_spk + ((unsigned long long)b * tslots + rslot) * g.num_trg;
    const unsigned int sslots = g.src_delay_slots;
    const float *stPre = g.src_spike_times +
        ((unsigned long long)b * sslots + ringSlot(k + sslots - g.axonal_delay, sslots)) * g.num_src;
    const float t = B200_FMUL((float)L.state->timestep, L.dt);
    const bool sparse = (g.connectivity == B200_CONN_SPARSE);
    const unsigned long long perBatch = sparse ? (unsigned long long)g.num_src * g.row_stride
                                               : (unsigned long long)g.num_src * g.num_trg;
    float *gb = g.g + (unsigned long long)b * perBatch;
    const unsigned int i = tile * POST_BLOCK + threadIdx.x;

    for(unsigned int s = blockIdx.y; s < count; s += gridDim.y) {
        const unsigned int post = spk[s];
        const unsigned int npre = sparse ? __ldg(&g.col_length[post]) : g.num_src;
        if(i >= npre) continue;
        unsigned long long idSyn;
        unsigned int pre;
        if(sparse) {
            idSyn = __ldg(&g.remap[(unsigned long long)post * g.col_stride + i]);
            pre = (unsigned int)(idSyn / g.row_stride);
        }
        else {
            pre = i;
            idSyn = (unsigned long long)i * g.num_trg + post;
        }
        const float dts = B200_FSUB(t, B200_FADD(g.wu_params[6], stPre[pre]));
        if(dts > 0.0f) {
            const float timing = expf(B200_FDIV(-dts, g.wu_params[0]));
            const float nw = B200_FADD(gb[idSyn], B200_FMUL(g.wu_params[2], timing));
            gb[idSyn] = fmaxf(g.wu_params[4], fminf(g.wu_params[5], nw));
        }
    }
}

// The non-zero words of a spike-recording array, as (word index + base, word) pairs appended to `pairs`
// (`counter` counts them all, also those beyond `capacity`).  A recording is one bit per neuron and time step and
// almost all zeros at cortical rates: the host fetches the pairs instead of the array (two per cent of its bytes
// at 3 Hz and dt = 0.1 ms).
__global__ void __launch_bounds__(256)
compactWordsKernel(const unsigned int *__restrict__ words, unsigned long long numWords, unsigned int base,
                   uint2 *__restrict__ pairs, unsigned int capacity, unsigned int *counter)
{
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < numWords; i += stride) {
        const unsigned int w = __ldg(&words[i]);
        if(w) {
            const unsigned int pos = atomicAdd(counter, 1u);
            if(pos < capacity) pairs[pos] = make_uint2(base + (unsigned int)i, w);
        }
    }
}

constexpr int REDUCE_BLOCK = 256;

// `phases`: bit 0 reduce, bit 1 write back.  Both in one pass on one GPU.  A data-parallel run reduces
// into `staged` (a segment of the buffer that one all-reduce combines over the processes), and in a
// second pass takes the combined value from there, stores it as the target and writes it back.
__global__ void __launch_bounds__(REDUCE_BLOCK)
batchReduceKernel(const b200_custom_update_group u, unsigned int batch, unsigned int phases, float *staged)
{
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long e = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; e < u.num_elements; e += stride) {
        float acc;
        if(phases & 1u) {
            acc = (u.op == B200_REDUCE_SUM) ? 0.0f : -3.402823466e+38f;
            for(unsigned int b = 0; b < batch; b++) {
                const float v = u.source[(unsigned long long)b * u.num_elements + e];
                acc = (u.op == B200_REDUCE_SUM) ? B200_FADD(acc, v) : fmaxf(acc, v);
            }
            (staged ? staged : u.target)[e] = acc;
        }
        else {
            acc = staged ? staged[e] : u.target[e];
            if(staged) u.target[e] = acc;
        }
        if(u.broadcast && (phases & 2u)) {
            const float w = B200_FMUL(acc, u.scale);
            for(unsigned int b = 0; b < batch; b++) u.source[(unsigned long long)b * u.num_elements + e] = w;
        }
    }
}
}   // namespace b200
