// Initialisation kernels: variable initialisation snippets, device-side sparse
// connectivity construction, per-synapse variable initialisation and the
// column-major remap.  Replace initializeKernel / initializeSparseKernel
// (backendSIMT.cc:1368-1779) for the built-in snippets
// (initVarSnippet.h:87-212, initSparseConnectivitySnippet.h:170-410).
//
// Every element draws from its own Philox stream keyed on (seed, stream id,
// element index), so the result does not depend on launch geometry and a CPU
// checker can regenerate any element independently.
#pragma once

#include "common.cuh"

namespace b200
{
constexpr int INIT_BLOCK = 256;

// One draw of a variable-initialisation snippet (initVarSnippet.h:87-212).
__host__ __device__ __forceinline__ float drawInitValue(unsigned int snippet, const float *p, b200_rng *rng)
{
    switch(snippet) {
    case B200_INIT_CONSTANT:
        return p[0];
    case B200_INIT_UNIFORM:
        return B200_FADD(p[0], B200_FMUL(b200_rng_uniform(rng), B200_FSUB(p[1], p[0])));
    case B200_INIT_NORMAL:
        return B200_FADD(p[0], B200_FMUL(b200_rng_normal(rng), p[1]));
    case B200_INIT_NORMAL_CLIPPED: {
        float v;
        do {
            v = B200_FADD(p[0], B200_FMUL(b200_rng_normal(rng), p[1]));
        } while(v > p[3] || v < p[2]);
        return v;
    }
    default: {      // B200_INIT_NORMAL_CLIPPED_DELAY: parameters already in time steps
        float v;
        do {
            v = B200_FADD(p[0], B200_FMUL(b200_rng_normal(rng), p[1]));
        } while(v > p[3] || v < p[2]);
        return rintf(v);
    }
    }
}

struct InitParams { float p[4]; };

template<typename T>
__global__ void __launch_bounds__(INIT_BLOCK)
initVarKernel(T *out, unsigned long long count, unsigned int snippet, InitParams prm,
              unsigned long long seed, unsigned int stream)
{
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long e = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += stride) {
        b200_rng rng = b200_rng_init(seed, stream, e);
        out[e] = (T)drawInitValue(snippet, prm.p, &rng);
    }
}

// Per-synapse variable over ragged rows: element index = pre*row_stride + j,
// drawn only where j < row_length[pre] (backendSIMT.h:414-469).
template<typename T>
__global__ void __launch_bounds__(INIT_BLOCK)
initSparseVarKernel(T *out, const unsigned int *__restrict__ row_length, unsigned int num_src,
                    unsigned int row_stride, unsigned int snippet, InitParams prm,
                    unsigned long long seed, unsigned int stream)
{
    const unsigned long long total = (unsigned long long)num_src * row_stride;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long e = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const unsigned int pre = (unsigned int)(e / row_stride);
        const unsigned int j = (unsigned int)(e - (unsigned long long)pre * row_stride);
        if(j < __ldg(&row_length[pre])) {
            b200_rng rng = b200_rng_init(seed, stream, e);
            out[e] = (T)drawInitValue(snippet, prm.p, &rng);
        }
        else {
            out[e] = (T)0;
        }
    }
}

template<typename IndT>
__device__ __forceinline__ void storeInd(void *ind, unsigned long long idx, unsigned int v)
{
    static_cast<IndT*>(ind)[idx] = (IndT)v;
}

// Row-build connectivity: one thread per presynaptic row
// (backendSIMT.cc:1606-1615).  Targets are drawn inside [trg_begin, trg_end)
// so a process that owns a slice of the target population builds only its own
// sub-matrix (the snippets' id_post_begin / num_post mechanism).
//   FixedProbability: geometric gaps, prevJ += 1 + (int)(log(u) / log(1-p))
//     (initSparseConnectivitySnippet.h:175-186); row_length is an output.
//   FixedNumberTotalWithReplacement: row_length is an INPUT (drawn on the host
//     from the multinomial, :300-336); targets ascend by sampling successive
//     first-order statistics x += (1-x)*(1 - u^(1/c)) (:283-291).
//   FixedNumberPostWithReplacement: `num` ascending targets per row likewise.
// The targets of one presynaptic row, in row order: emit(n, target) for n = 0, 1, ...; returns how
// many there are.  One Philox stream per row, so a row can be regenerated at any time from
// (seed, stream, pre): the initialisation kernel below stores what this yields, the PROCEDURAL
// presynaptic kernel (presynaptic_update.cuh) replays it for every spike.  `fixedLength` is the
// row length for the snippets that take it as an input.
//
// Sub-rows (FixedProbability only, p[2] = T > 1; the reference's "threads per spike",
// presynapticUpdateStrategySIMT.cc:425-561): the targets are cut into T equal ranges and the synapses
// into range t are drawn from a stream of their own, element pre * T + t, so T threads can regenerate
// one row side by side.  The row is the sub-rows one after the other; [subFirst, subLast) selects
// which of them to generate (n then counts from the first one generated).
__host__ __device__ __forceinline__ unsigned int connectSubRows(unsigned int snippet, const float *p)
{
    const bool prob = (snippet == B200_CONNECT_FIXED_PROBABILITY || snippet == B200_CONNECT_FIXED_PROBABILITY_NO_AUTAPSE);
    return (prob && p[2] > 1.0f) ? (unsigned int)p[2] : 1u;
}

template<typename F>
__host__ __device__ __forceinline__ unsigned int generateRow(unsigned int snippet, const float *p, unsigned int pre,
                                                             unsigned int trg_begin, unsigned int trg_end,
                                                             unsigned int fixedLength, unsigned long long seed,
                                                             unsigned int stream, F emit,
                                                             unsigned int subFirst = 0u, unsigned int subLast = 0xFFFFFFFFu)
{
    const unsigned int numPost = trg_end - trg_begin;
    unsigned int n = 0;
    if(snippet == B200_CONNECT_FIXED_PROBABILITY || snippet == B200_CONNECT_FIXED_PROBABILITY_NO_AUTAPSE) {
        const float probLogRecip = p[1];       // 1 / log(1 - prob), computed on the host in double
        const unsigned int T = connectSubRows(snippet, p);
        const unsigned int per = (numPost + T - 1u) / T;
        for(unsigned int t = subFirst; t < T && t < subLast; t++) {
            const unsigned int lo = t * per;
            if(lo >= numPost) break;
            const unsigned int span = min(per, numPost - lo);
            b200_rng rng = b200_rng_init(seed, stream, (unsigned long long)pre * T + t);
            int prevJ = -1;
            while(true) {
                const float u = b200_rng_uniform(&rng);
                prevJ += 1 + (int)B200_FMUL(b200_logf(u), probLogRecip);
                if(snippet == B200_CONNECT_FIXED_PROBABILITY_NO_AUTAPSE && (unsigned int)prevJ + lo + trg_begin == pre) continue;
                if(prevJ >= 0 && (unsigned int)prevJ < span) {
                    emit(n, (unsigned int)prevJ + lo + trg_begin);
                    n++;
                }
                else {
                    break;
                }
            }
        }
    }
    else {
        b200_rng rng = b200_rng_init(seed, stream, pre);
        float x = 0.0f;
        for(unsigned int c = fixedLength; c != 0; c--) {
            const float u = b200_rng_uniform(&rng);
            // 1 - u^(1/c) with u^(1/c) = exp(log(u)/c)
            const float root = b200_expf(B200_FDIV(b200_logf(u), (float)c));
            x = B200_FADD(x, B200_FMUL(B200_FSUB(1.0f, x), B200_FSUB(1.0f, root)));
            unsigned int postIdx = (unsigned int)B200_FMUL(x, (float)numPost);
            postIdx = (postIdx < numPost) ? postIdx : (numPost - 1);
            emit(n, postIdx + trg_begin);
            n++;
        }
    }
    return n;
}

template<typename IndT>
__global__ void __launch_bounds__(INIT_BLOCK)
initSparseConnectivityKernel(unsigned int snippet, InitParams prm, unsigned int num_src,
                             unsigned int row_stride, unsigned int trg_begin, unsigned int trg_end,
                             unsigned int *row_length, void *ind, unsigned long long seed, unsigned int stream,
                             StepState *state)
{
    const unsigned int pre = blockIdx.x * blockDim.x + threadIdx.x;
    if(pre >= num_src) return;
    const unsigned long long base = (unsigned long long)pre * row_stride;
    const bool lengthIsOutput = (snippet == B200_CONNECT_FIXED_PROBABILITY || snippet == B200_CONNECT_FIXED_PROBABILITY_NO_AUTAPSE);
    unsigned int c = 0;
    if(!lengthIsOutput) {
        c = (snippet == B200_CONNECT_FIXED_NUMBER_POST_WITH_REPLACEMENT) ? (unsigned int)prm.p[0] : row_length[pre];
        if(c > row_stride) {
            atomicOr(&state->error, ERR_IND_RANGE);
            c = row_stride;
        }
    }
    unsigned int n = generateRow(snippet, prm.p, pre, trg_begin, trg_end, c, seed, stream,
                                 [&](unsigned int at, unsigned int target) {
                                     if(at < row_stride) storeInd<IndT>(ind, base + at, target);
                                 });
    if(n > row_stride) {
        atomicOr(&state->error, ERR_IND_RANGE);
        n = row_stride;
    }
    if(lengthIsOutput || snippet == B200_CONNECT_FIXED_NUMBER_POST_WITH_REPLACEMENT) row_length[pre] = n;
}

// Column-build connectivity with a fixed in-degree: one thread per target
// neuron appends `num` synapses to uniformly drawn rows with an atomic on the
// row length (backendSIMT.cc:1617-1623;
// initSparseConnectivitySnippet.h:376-384).  The order of synapses inside a
// row depends on the atomics; the multiset of (pre, post) pairs does not.
template<typename IndT>
__global__ void __launch_bounds__(INIT_BLOCK)
initFixedNumberPreKernel(unsigned int num, unsigned int num_src, unsigned int row_stride,
                         unsigned int trg_begin, unsigned int trg_end, unsigned int *row_length, void *ind,
                         unsigned long long seed, unsigned int stream, StepState *state)
{
    const unsigned int post = trg_begin + blockIdx.x * blockDim.x + threadIdx.x;
    if(post >= trg_end) return;
    b200_rng rng = b200_rng_init(seed, stream, post);
    for(unsigned int c = 0; c < num; c++) {
        const unsigned int pre = b200_rng_u32(&rng) % num_src;
        const unsigned int pos = atomicAdd(&row_length[pre], 1u);
        if(pos < row_stride) {
            storeInd<IndT>(ind, (unsigned long long)pre * row_stride + pos, post);
        }
        else {
            atomicOr(&state->error, ERR_IND_RANGE);
        }
    }
}

// Column lengths and column-major remap of ragged rows (genRemap,
// backendSIMT.cc:1977-1991): thread per synapse slot, atomicAdd on the column.
template<typename IndT>
__global__ void __launch_bounds__(INIT_BLOCK)
buildRemapKernel(const unsigned int *__restrict__ row_length, const void *__restrict__ ind,
                 unsigned int num_src, unsigned int num_trg, unsigned int row_stride, unsigned int col_stride,
                 unsigned int *col_length, unsigned int *remap, StepState *state)
{
    const unsigned long long total = (unsigned long long)num_src * row_stride;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for(unsigned long long e = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const unsigned int pre = (unsigned int)(e / row_stride);
        const unsigned int j = (unsigned int)(e - (unsigned long long)pre * row_stride);
        if(j < __ldg(&row_length[pre])) {
            const unsigned int post = static_cast<const IndT*>(ind)[e];
            if(post >= num_trg) {
                atomicOr(&state->error, ERR_IND_RANGE);
                continue;
            }
            const unsigned int pos = atomicAdd(&col_length[post], 1u);
            if(pos < col_stride) {
                remap[(unsigned long long)post * col_stride + pos] = (unsigned int)e;
            }
            else {
                atomicOr(&state->error, ERR_IND_RANGE);
            }
        }
    }
}
}   // namespace b200
