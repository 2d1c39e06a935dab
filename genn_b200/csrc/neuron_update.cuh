// Neuron update kernel: postsynaptic models, current sources, neuron dynamics,
// threshold, reset, spike emission and recording for every merged neuron group
// in one launch.  Replaces the reference's neuronSpikeQueueUpdateKernel +
// updateNeuronsKernel pair (backendSIMT.cc:373-662) and the per-group code of
// NeuronUpdateGroupMerged::generateNeuronUpdate
// (neuronUpdateGroupMerged.cc:552-773).
//
// Layout: one thread per neuron, groups padded to whole blocks, grid.y = batch.
// All state is SoA fp32 so every load/store is a coalesced 128-byte line per
// warp.  Spikes are compacted with a warp ballot and ONE atomicAdd per warp
// that spiked (the reference stages ids in shared memory and issues one atomic
// per block per step whether or not anything spiked).  The same ballot word is
// the 32-neuron spike-recording word, written with a plain store.  The last
// block to finish (ticket) clears the spike counts of the slot the next step
// will write and advances the step counters, which is what the reference's
// separate one-thread-per-group queue-update kernel does.
//
// Arithmetic uses single IEEE operations without fused contraction in the
// order of the reference's model strings (neuronModels.h:168-241,
// postsynapticModels.h:98-148, currentSourceModels.h:111-122) so results are
// bit-identical to the CPU backend for identical inputs.
#pragma once

#include "common.cuh"

namespace b200
{
constexpr int NEURON_BLOCK = 128;

struct NeuronLaunch
{
    const b200_neuron_group *groups;
    const unsigned int *block_start;
    unsigned int num_groups;
    unsigned int batch;
    float dt;
    unsigned long long seed;
    unsigned long long num_recording_timesteps;
    StepState *state;
    unsigned int count_events;
};

__global__ void __launch_bounds__(NEURON_BLOCK)
neuronUpdateKernel(const NeuronLaunch L)
{
    const unsigned int gi = findGroup(L.block_start, L.num_groups, blockIdx.x);
    const b200_neuron_group &g = L.groups[gi];
    const unsigned int b = blockIdx.y;
    const unsigned int N = g.num_neurons;
    const unsigned int local = (blockIdx.x - __ldg(&L.block_start[gi])) * NEURON_BLOCK + threadIdx.x;
    const unsigned int i = g.first_neuron + local;
    const bool active = local < g.num_update;

    const unsigned long long k = L.state->steps_done;
    const unsigned long long timestep = L.state->timestep;
    const float t = B200_FMUL((float)timestep, L.dt);
    const unsigned int slots = g.num_delay_slots;
    const unsigned int wslot = ringSlot(k + 1, slots);
    const unsigned long long bi = (unsigned long long)b * N + i;

    bool spiked = false;
    if(active) {
        float Isyn = 0.0f;
        float V = 0.0f;
        const unsigned int model = g.model;
        if(model == B200_NEURON_LIF || model == B200_NEURON_IZHIKEVICH) {
            V = static_cast<float*>(g.vars[0])[bi];
        }

        // incoming fused postsynaptic models
        const unsigned int numPSM = g.num_psm;
        for(unsigned int p = 0; p < numPSM; p++) {
            const b200_psm &psm = g.psm[p];
            float linSyn = psm.out_post[bi];
            const unsigned int D = psm.max_den_delay;
            if(D) {
                float *front = &psm.den_delay[((unsigned long long)b * D + ringSlot(k + 1, D)) * N + i];
                linSyn = B200_FADD(linSyn, *front);
                *front = 0.0f;
            }
            if(psm.model == B200_PSM_EXP_CURR) {
                Isyn = B200_FADD(Isyn, B200_FMUL(psm.params[0], linSyn));
                linSyn = B200_FMUL(linSyn, psm.params[1]);
            }
            else if(psm.model == B200_PSM_EXP_COND) {
                Isyn = B200_FADD(Isyn, B200_FMUL(linSyn, B200_FSUB(psm.params[1], V)));
                linSyn = B200_FMUL(linSyn, psm.params[0]);
            }
            else {
                Isyn = B200_FADD(Isyn, linSyn);
                linSyn = 0.0f;
            }
            psm.out_post[bi] = linSyn;
        }

        // current sources
        const unsigned int numCS = g.num_cs;
        for(unsigned int c = 0; c < numCS; c++) {
            const b200_current_source &cs = g.cs[c];
            if(cs.model == B200_CS_DC) {
                Isyn = B200_FADD(Isyn, cs.params[0]);
            }
            else {
                float current = cs.var0[bi];
                b200_rng rng = b200_rng_sim(L.seed, cs.rng_stream, b * N + i, timestep);
                float p = 1.0f;
                unsigned int numSpikes = 0;
                const float expMinusLambda = cs.params[2];
                do {
                    numSpikes++;
                    p = B200_FMUL(p, b200_rng_uniform(&rng));
                } while(p > expMinusLambda);
                current = B200_FADD(current, B200_FMUL(cs.params[0], (float)(numSpikes - 1)));
                Isyn = B200_FADD(Isyn, current);
                current = B200_FMUL(current, cs.params[1]);
                cs.var0[bi] = current;
            }
        }

        if(model == B200_NEURON_LIF) {
            float R = static_cast<float*>(g.vars[1])[bi];
            if(R <= 0.0f) {
                const float alpha = B200_FADD(B200_FMUL(B200_FADD(Isyn, g.params[3]), g.params[4]), g.params[2]);
                V = B200_FSUB(alpha, B200_FMUL(g.params[5], B200_FSUB(alpha, V)));
            }
            else {
                R = B200_FSUB(R, L.dt);
            }
            if(R <= 0.0f && V >= g.params[0]) {
                spiked = true;
                V = g.params[1];
                R = g.params[6];
            }
            static_cast<float*>(g.vars[0])[bi] = V;
            static_cast<float*>(g.vars[1])[bi] = R;
        }
        else if(model == B200_NEURON_IZHIKEVICH) {
            float U = static_cast<float*>(g.vars[1])[bi];
            const float dt = L.dt;
            if(V >= 30.0f) {
                V = g.params[2];
                U = B200_FADD(U, g.params[3]);
            }
            for(int half = 0; half < 2; half++) {
                // 0.04*V*V + 5*V + 140 - U + Isyn, left to right
                float x = B200_FMUL(B200_FMUL(0.04f, V), V);
                x = B200_FADD(x, B200_FMUL(5.0f, V));
                x = B200_FADD(x, 140.0f);
                x = B200_FSUB(x, U);
                x = B200_FADD(x, Isyn);
                V = B200_FADD(V, B200_FMUL(B200_FMUL(0.5f, x), dt));
            }
            U = B200_FADD(U, B200_FMUL(B200_FMUL(g.params[0], B200_FSUB(B200_FMUL(g.params[1], V), U)), dt));
            if(V > 30.0f) V = 30.0f;
            spiked = (V >= 29.99f);
            static_cast<float*>(g.vars[0])[bi] = V;
            static_cast<float*>(g.vars[1])[bi] = U;
        }
        else if(model == B200_NEURON_SPIKE_SOURCE_ARRAY) {
            unsigned int start = static_cast<unsigned int*>(g.vars[0])[bi];
            const unsigned int end = static_cast<const unsigned int*>(g.vars[1])[bi];
            if(start != end && t >= __ldg(&g.egp[start])) {
                spiked = true;
                static_cast<unsigned int*>(g.vars[0])[bi] = start + 1;
            }
        }
        else {
            float tts = static_cast<float*>(g.vars[0])[bi];
            if(tts <= 0.0f) {
                b200_rng rng = b200_rng_sim(L.seed, g.rng_stream, b * N + i, timestep);
                tts = B200_FADD(tts, B200_FMUL(g.params[0], -b200_logf(b200_rng_uniform(&rng))));
            }
            tts = B200_FSUB(tts, 1.0f);
            spiked = (tts <= 0.0f);
            static_cast<float*>(g.vars[0])[bi] = tts;
        }
    }

    // ---- spike emission: ballot + one atomic per spiking warp ----------------
    const unsigned int ballot = __ballot_sync(0xFFFFFFFFu, spiked);
    const unsigned int lane = threadIdx.x & 31u;
    if(ballot) {
        unsigned int base = 0;
        if(lane == 0) {
            base = atomicAdd(&g.spk_cnt[b * slots + wslot], __popc(ballot));
        }
        base = __shfl_sync(0xFFFFFFFFu, base, 0);
        if(L.count_events && lane == 0) atomicAdd(&L.state->spikes, (unsigned long long)__popc(ballot));
        if(spiked) {
            const unsigned int pos = base + __popc(ballot & ((1u << lane) - 1u));
            if(pos < N) {
                g.spk[((unsigned long long)b * slots + wslot) * N + pos] = i;
            }
            else {
                atomicOr(&L.state->error, ERR_SPIKE_OVERFLOW);
            }
        }
    }
    // spike times ride in the queue: carry the previous slot forward
    if(g.spike_times && active) {
        float *st = g.spike_times + ((unsigned long long)b * slots) * N;
        st[(unsigned long long)wslot * N + i] = spiked ? t : st[(unsigned long long)ringSlot(k, slots) * N + i];
    }
    // recording: bit i%32 of word i/32 (backendSIMT.cc:617-660)
    if(g.record_spk && L.num_recording_timesteps) {
        const unsigned int words = (N + 31u) / 32u;
        unsigned int *rec = g.record_spk + ((timestep % L.num_recording_timesteps) * L.batch + b) * words;
        // first_neuron is a multiple of 32, so a warp covers exactly one word
        if(lane == 0 && local < ((g.num_update + 31u) & ~31u) && (i / 32u) < words) rec[i / 32u] = ballot;
    }

    // ---- last block: queue update for the next step and counter advance -------
    __shared__ bool isLast;
    __threadfence();
    __syncthreads();
    if(threadIdx.x == 0) {
        const unsigned int total = gridDim.x * gridDim.y;
        isLast = (atomicAdd(&L.state->ticket, 1u) == total - 1u);
    }
    __syncthreads();
    if(isLast) {
        for(unsigned int q = threadIdx.x; q < L.num_groups * L.batch; q += blockDim.x) {
            const b200_neuron_group &o = L.groups[q / L.batch];
            const unsigned int ob = q % L.batch;
            o.spk_cnt[ob * o.num_delay_slots + ringSlot(k + 2, o.num_delay_slots)] = 0;
        }
        if(threadIdx.x == 0) {
            L.state->ticket = 0;
            L.state->timestep = timestep + 1;
            L.state->steps_done = k + 1;
            __threadfence();
        }
    }
}
}   // namespace b200
