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

// Peers of a sharded model as the neuron update sees them: every spike id is also
// stored into each peer's exchange arena, at the offset it has in this process's.
struct ExchangeCtx
{
    unsigned int world;
    unsigned int rank;
    unsigned char *arena;
    unsigned char *const *peers;        // [B200_MAX_RANKS], shared or global memory
    unsigned long long tag;             // step number the words of this step carry in their high half
};

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

// Loads of data other SMs write between grid barriers (postsynaptic input,
// spike times) must come from L2 when the kernel persists across time steps.
template<bool COHERENT, typename T>
__device__ __forceinline__ T loadShared(const T *p)
{
    return COHERENT ? __ldcg(p) : *p;
}

// Everything one neuron carries from step to step, as registers: the model's
// two state variables (bit patterns: SpikeSourceArray keeps integers), the
// running input of each fused postsynaptic model and each current source's
// variable.  Loading it as one batch of independent loads, before any store,
// keeps a single memory round trip on the critical path; the persistent kernel
// keeps it in registers across steps.
// NPSM / NCS bound the number of fused postsynaptic models and current sources
// of any group the kernel instance handles: the host picks the smallest
// instance that covers the model, so the unrolled loops below carry no dead
// iterations (a Potjans group has one of each).
template<int NPSM, int NCS>
struct NeuronRegs
{
    unsigned int v[2];
    float lin[NPSM];
    float cs[NCS > 0 ? NCS : 1];
};

__device__ __forceinline__ bool modelHasVar1(unsigned int model)
{
    return model != B200_NEURON_POISSON;
}

template<bool COHERENT, int NPSM, int NCS>
__device__ __forceinline__ void loadNeuron(const b200_neuron_group &g, unsigned long long bi, NeuronRegs<NPSM, NCS> &r)
{
    r.v[0] = static_cast<const unsigned int*>(g.vars[0])[bi];
    r.v[1] = modelHasVar1(g.model) ? static_cast<const unsigned int*>(g.vars[1])[bi] : 0u;
    #pragma unroll
    for(unsigned int p = 0; p < NPSM; p++) {
        r.lin[p] = (p < g.num_psm) ? loadShared<COHERENT>(&g.psm[p].out_post[bi]) : 0.0f;
    }
    #pragma unroll
    for(unsigned int c = 0; c < NCS; c++) {
        r.cs[c] = (c < g.num_cs && g.cs[c].var0) ? g.cs[c].var0[bi] : 0.0f;
    }
}

template<int NPSM, int NCS>
__device__ __forceinline__ void storeNeuron(const b200_neuron_group &g, unsigned long long bi,
                                            const NeuronRegs<NPSM, NCS> &r, bool onlyPrivate)
{
    static_cast<unsigned int*>(g.vars[0])[bi] = r.v[0];
    if(modelHasVar1(g.model) && g.model != B200_NEURON_SPIKE_SOURCE_ARRAY) static_cast<unsigned int*>(g.vars[1])[bi] = r.v[1];
    #pragma unroll
    for(unsigned int p = 0; p < NPSM; p++) {
        // inputs without a dendritic-delay ring receive reductions directly and
        // are written back every step by the caller
        if(p < g.num_psm && (!onlyPrivate || g.psm[p].max_den_delay)) g.psm[p].out_post[bi] = r.lin[p];
    }
    #pragma unroll
    for(unsigned int c = 0; c < NCS; c++) {
        if(c < g.num_cs && g.cs[c].var0) g.cs[c].var0[bi] = r.cs[c];
    }
}

// Front slot of every dendritic-delay ring: read and cleared
// (neuronUpdateGroupMerged.cc:96-113).
template<bool COHERENT, int NPSM>
__device__ __forceinline__ void takeFronts(const b200_neuron_group &g, unsigned int b, unsigned int i,
                                           unsigned int k, float (&front)[NPSM])
{
    // every load before any store: the pointers are generic, so a store between
    // two loads would force the second load to wait for the first
    float *slot[NPSM];
    #pragma unroll
    for(unsigned int p = 0; p < NPSM; p++) {
        front[p] = 0.0f;
        slot[p] = nullptr;
        if(p < g.num_psm) {
            const unsigned int D = g.psm[p].max_den_delay;
            if(D) {
                slot[p] = &g.psm[p].den_delay[((unsigned long long)b * D + ringSlot(k + 1, D)) * g.num_neurons + i];
                front[p] = loadShared<COHERENT>(slot[p]);
            }
        }
    }
    #pragma unroll
    for(unsigned int p = 0; p < NPSM; p++) {
        if(slot[p]) *slot[p] = 0.0f;
    }
}

// One neuron, one time step, entirely in registers.  Returns whether it spiked.
// Random draws of the current sources for one neuron and step: the number of
// Poisson events of each PoissonExp source.  They depend on nothing the
// presynaptic phase produces, so the persistent kernel computes them while the
// barrier after that phase is in flight.
// The model draws its Poisson count by multiplying uniforms until the product
// falls below exp(-lambda) (currentSourceModels.h:111-118); here the same count
// comes from inverting the Poisson CDF with one uniform, a quarter of a Philox
// block per step instead of one or two whole blocks.
template<int NCS>
__device__ __forceinline__ void drawCurrentSources(const NeuronLaunch &L, const b200_neuron_group &g, unsigned int b,
                                                   unsigned int i, unsigned long long timestep,
                                                   unsigned int (&count)[NCS > 0 ? NCS : 1])
{
    #pragma unroll
    for(unsigned int c = 0; c < NCS; c++) {
        count[c] = 0;
        if(c < g.num_cs && g.cs[c].model == B200_CS_POISSON_EXP) {
            const b200_current_source &cs = g.cs[c];
            const b200_philox_out blk = b200_rng_step_block(L.seed, cs.rng_stream, b * g.num_neurons + i, timestep);
            const float u = b200_u32_to_uniform(b200_rng_step_word(&blk, timestep));
            count[c] = b200_poisson_inverse(u, cs.params[2], cs.params[3]);
        }
    }
}

template<int NPSM, int NCS>
__device__ __forceinline__ bool neuronCompute(const NeuronLaunch &L, const b200_neuron_group &g, unsigned int b,
                                              unsigned int i, unsigned long long timestep, float t,
                                              NeuronRegs<NPSM, NCS> &r, const float (&front)[NPSM],
                                              const unsigned int (&csCount)[NCS > 0 ? NCS : 1])
{
    const unsigned int N = g.num_neurons;
    const unsigned int model = g.model;
    float Isyn = 0.0f;
    float V = __uint_as_float(r.v[0]);

    // incoming fused postsynaptic models
    #pragma unroll
    for(unsigned int p = 0; p < NPSM; p++) {
        if(p < g.num_psm) {
            const b200_psm &psm = g.psm[p];
            float linSyn = B200_FADD(r.lin[p], front[p]);
            if(!psm.max_den_delay) linSyn = r.lin[p];
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
            r.lin[p] = linSyn;
        }
    }

    // current sources
    #pragma unroll
    for(unsigned int c = 0; c < NCS; c++) {
        if(c < g.num_cs) {
            const b200_current_source &cs = g.cs[c];
            if(cs.model == B200_CS_DC) {
                Isyn = B200_FADD(Isyn, cs.params[0]);
            }
            else {
                float current = r.cs[c];
                current = B200_FADD(current, B200_FMUL(cs.params[0], (float)csCount[c]));
                Isyn = B200_FADD(Isyn, current);
                r.cs[c] = B200_FMUL(current, cs.params[1]);
            }
        }
    }

    bool spiked = false;
    if(model == B200_NEURON_LIF) {
        float R = __uint_as_float(r.v[1]);
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
        r.v[0] = __float_as_uint(V);
        r.v[1] = __float_as_uint(R);
    }
    else if(model == B200_NEURON_IZHIKEVICH) {
        float U = __uint_as_float(r.v[1]);
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
        r.v[0] = __float_as_uint(V);
        r.v[1] = __float_as_uint(U);
    }
    else if(model == B200_NEURON_SPIKE_SOURCE_ARRAY) {
        const unsigned int start = r.v[0], end = r.v[1];
        if(start != end && t >= __ldg(&g.egp[start])) {
            spiked = true;
            r.v[0] = start + 1;
        }
    }
    else {
        float tts = V;
        if(tts <= 0.0f) {
            b200_rng rng = b200_rng_sim(L.seed, g.rng_stream, b * N + i, timestep);
            tts = B200_FADD(tts, B200_FMUL(g.params[0], -b200_logf(b200_rng_uniform(&rng))));
        }
        tts = B200_FSUB(tts, 1.0f);
        spiked = (tts <= 0.0f);
        r.v[0] = __float_as_uint(tts);
    }
    return spiked;
}

// Spike emission (ballot + one atomic per spiking warp), spike times and
// recording.  Called by whole warps.
template<bool COHERENT>
__device__ __forceinline__ void neuronEmit(const NeuronLaunch &L, const b200_neuron_group &g, unsigned int b,
                                           unsigned int local, bool spiked, unsigned int k,
                                           unsigned long long timestep, float t, const ExchangeCtx *x = nullptr)
{
    const unsigned int N = g.num_neurons;
    const unsigned int i = g.first_neuron + local;
    const bool active = local < g.num_update;
    const unsigned int slots = g.num_delay_slots;
    const unsigned int wslot = ringSlot(k + 1, slots);
    const unsigned int listStride = g.spk_slot_stride ? g.spk_slot_stride : N;
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
            if(pos < listStride) {
                unsigned int *cell = &g.spk[((unsigned long long)b * slots + wslot) * listStride + pos];
                *cell = i;
                if(x) {
                    // the travelling copy: (step << 32 | id) into the same cell of every
                    // process's arena, this one included.  Each word validates itself,
                    // so the stores need no ordering and nothing waits for them.
                    unsigned long long *wire = reinterpret_cast<unsigned long long*>(g.spk_wire) +
                                               ((unsigned long long)b * slots + wslot) * listStride + pos;
                    const unsigned long long word = (x->tag << 32) | (unsigned long long)i;
                    for(unsigned int p = 0; p < x->world; p++) {
                        unsigned long long *dst = (p == x->rank) ? wire
                            : reinterpret_cast<unsigned long long*>(x->peers[p] + (reinterpret_cast<unsigned char*>(wire) - x->arena));
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(dst), "l"(word) : "memory");
                    }
                }
            }
            else {
                atomicOr(&L.state->error, ERR_SPIKE_OVERFLOW);
            }
        }
    }
    // spike times ride in the queue: carry the previous slot forward
    if(g.spike_times && active) {
        float *st = g.spike_times + ((unsigned long long)b * slots) * N;
        st[(unsigned long long)wslot * N + i] = spiked ? t : loadShared<COHERENT>(&st[(unsigned long long)ringSlot(k, slots) * N + i]);
    }
    // recording: the updated slice only, bit j%32 of word j/32 for its j-th neuron
    // (backendSIMT.cc:617-660 for a whole population)
    if(g.record_spk && L.num_recording_timesteps) {
        const unsigned int words = (g.num_update + 31u) / 32u;
        // a warp covers exactly one word; only the writing lane pays for the 64-bit modulo
        if(lane == 0 && (local / 32u) < words) {
            unsigned int *rec = g.record_spk + ((timestep % L.num_recording_timesteps) * L.batch + b) * words;
            rec[local / 32u] = ballot;
        }
    }
}

// One neuron, one time step with its state in global memory: called by whole
// warps (`local` may lie past the end of the group; such lanes only take part in
// the ballot).  `k` is the number of completed steps, `timestep` the model step.
template<bool COHERENT, int NPSM, int NCS>
__device__ __forceinline__ void neuronStep(const NeuronLaunch &L, const b200_neuron_group &g, unsigned int b,
                                           unsigned int local, unsigned int k, unsigned long long timestep,
                                           const ExchangeCtx *x = nullptr)
{
    const unsigned int i = g.first_neuron + local;
    const float t = B200_FMUL((float)timestep, L.dt);
    bool spiked = false;
    if(local < g.num_update) {
        const unsigned long long bi = (unsigned long long)b * g.num_neurons + i;
        NeuronRegs<NPSM, NCS> r;
        float front[NPSM];
        unsigned int csCount[NCS > 0 ? NCS : 1];
        loadNeuron<COHERENT>(g, bi, r);
        takeFronts<COHERENT, NPSM>(g, b, i, k, front);
        drawCurrentSources<NCS>(L, g, b, i, timestep, csCount);
        spiked = neuronCompute(L, g, b, i, timestep, t, r, front, csCount);
        storeNeuron(g, bi, r, false);
    }
    neuronEmit<COHERENT>(L, g, b, local, spiked, k, timestep, t, x);
}

template<int NPSM, int NCS>
__global__ void __launch_bounds__(NEURON_BLOCK)
neuronUpdateKernel(const NeuronLaunch L)
{
    const unsigned int gi = findGroup(L.block_start, L.num_groups, blockIdx.x);
    const b200_neuron_group &g = L.groups[gi];
    const unsigned int local = (blockIdx.x - __ldg(&L.block_start[gi])) * NEURON_BLOCK + threadIdx.x;
    const unsigned int k = L.state->phase;
    const unsigned long long timestep = L.state->timestep;
    neuronStep<false, NPSM, NCS>(L, g, blockIdx.y, local, k, timestep);

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
        __shared__ unsigned int stepSpikes;
        if(threadIdx.x == 0) stepSpikes = 0u;
        __syncthreads();
        for(unsigned int q = threadIdx.x; q < L.num_groups * L.batch; q += blockDim.x) {
            const b200_neuron_group &o = L.groups[q / L.batch];
            const unsigned int ob = q % L.batch;
            o.spk_cnt[ob * o.num_delay_slots + ringSlot(k + 2, o.num_delay_slots)] = 0;
            atomicAdd(&stepSpikes, __ldcg(&o.spk_cnt[ob * o.num_delay_slots + ringSlot(k + 1, o.num_delay_slots)]));
        }
        __syncthreads();
        if(threadIdx.x == 0) {
            atomicMax(&L.state->peak_spikes, stepSpikes);
            L.state->ticket = 0;
            L.state->timestep = timestep + 1;
            L.state->steps_done = L.state->steps_done + 1;
            L.state->phase = (k + 1 == L.state->ring_period) ? 0u : k + 1;
            __threadfence();
        }
    }
}
}   // namespace b200
