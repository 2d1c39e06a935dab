// b200_update_neurons_noalloc: one neuron update with every byte of scratch
// memory taken from a fixed array that is part of the library image.
//
// Who needs it.  The regular path (b200_push_neuron_update_group +
// b200_update_neurons) keeps device copies of the merged-group descriptors, a
// block lookup table and the step counters in memory it obtains with
// cudaMalloc.  Some hosts of this library must never allocate once they are
// running: a real-time control loop that closes a brain-machine or robot loop
// around a spiking model and cannot tolerate the unbounded latency (or the
// implicit device synchronisation) of an allocator call; a plugin living inside
// somebody else's process whose memory budget was fixed at start-up and whose
// owner forbids further device allocations.  For them this entry point does the
// same neuron update with its scratch in `g_scratch` below.
//
// What it costs.  Every GPU that loads the library carries the array
// (B200_NOALLOC_SCRATCH_BYTES, 40 KB) until the process exits, and the
// number of neuron groups per call is capped (B200_NOALLOC_MAX_GROUPS).
//
// Rules of use.
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, which may load the module).  Make that first call
//    before starting any stream capture.
//  * A call on a stream that is being captured is refused (B200_ERR_STATE):
//    every call copies its tables and counters from host memory that is gone
//    by the time a captured graph would replay.
//  * A kernel-side bounds check that fails (a spike list too short for the
//    spikes of the step) sets a word in the array.  b200_noalloc_check waits
//    for the stream and reports it; the next update clears it.
//  * The caller's current device is left as it was found.
//  * All calls on one device share the one array, and the array keeps what the
//    last call left in it.  Everything that must start from a known value (the
//    block ticket, the error word, the step counters) is rewritten by every
//    call, in stream order.  Two calls whose GPU work can overlap (different
//    streams without an ordering between them) race on the array: order them.
//  * The caller owns every array the descriptors point at (inputs and outputs)
//    and the stream.  Nothing is allocated or freed here, on the host or on the
//    device.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "genn_b200.h"
#include "common.cuh"
#include "neuron_update.cuh"

using namespace b200;

namespace
{
struct Scratch
{
    StepState state;
    unsigned int blockStart[B200_NOALLOC_MAX_GROUPS + 1];
    unsigned int pad[3];
    b200_neuron_group groups[B200_NOALLOC_MAX_GROUPS];
};
static_assert(sizeof(Scratch) <= B200_NOALLOC_SCRATCH_BYTES, "scratch layout exceeds the stated size");

// The scratch itself.  In host code this name is only a handle for the
// runtime's symbol table; it is never passed to a kernel.  The device address
// comes from cudaGetSymbolAddress (below).
static __device__ __align__(256) unsigned char g_scratch[B200_NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
unsigned char *g_scratchAddress[MAX_DEVICES] = {};
std::mutex g_setupMutex;

thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

// Once per device, with that device current: resolve the device address of the
// scratch array.
int scratchAddress(int device, unsigned char **out)
{
    std::lock_guard<std::mutex> lock(g_setupMutex);
    if(!g_scratchAddress[device]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
        if(e != cudaSuccess || !p) {
            return fail(B200_ERR_CUDA, "cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
        }
        g_scratchAddress[device] = static_cast<unsigned char*>(p);
    }
    *out = g_scratchAddress[device];
    return B200_OK;
}

// Makes `device` current for the length of a call and puts the caller's device back.
struct DeviceGuard
{
    int previous = -1;
    cudaError_t enter(int device)
    {
        cudaError_t e = cudaGetDevice(&previous);
        if(e != cudaSuccess) { previous = -1; return e; }
        if(previous == device) { previous = -1; return cudaSuccess; }
        return cudaSetDevice(device);
    }
    ~DeviceGuard() { if(previous >= 0) cudaSetDevice(previous); }
};

unsigned long long foldPeriod(unsigned long long period, unsigned int n)
{
    if(n < 2) return period;
    unsigned long long a = period, b = n;
    while(b) { const unsigned long long t = a % b; a = b; b = t; }
    return period / a * n;
}

template<int P, int C>
void launch(const NeuronLaunch &L, dim3 grid, cudaStream_t stream)
{
    neuronUpdateKernel<P, C><<<grid, NEURON_BLOCK, 0, stream>>>(L);
}
}   // anonymous namespace

extern "C" {

const char *b200_noalloc_last_error(void)
{
    return g_error;
}

int b200_update_neurons_noalloc(int device, void *stream, const b200_neuron_group *groups, uint32_t num_groups,
                                uint32_t batch_size, double dt, uint64_t seed, uint64_t timestep,
                                uint64_t steps_done, uint64_t num_recording_timesteps)
{
    if(!groups || num_groups == 0 || batch_size == 0) return fail(B200_ERR_INVALID, "no neuron groups given");
    if(num_groups > B200_NOALLOC_MAX_GROUPS) {
        return fail(B200_ERR_INVALID, "%u neuron groups exceed the limit of %u that fit the built-in scratch array",
                    num_groups, (unsigned int)B200_NOALLOC_MAX_GROUPS);
    }
    if(device < 0 || device >= MAX_DEVICES) return fail(B200_ERR_INVALID, "device index %d out of range", device);
    DeviceGuard guard;
    cudaError_t e = guard.enter(device);
    if(e != cudaSuccess) return fail(B200_ERR_CUDA, "cudaSetDevice(%d) failed: %s", device, cudaGetErrorString(e));
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &capture);
    if(e != cudaSuccess) return fail(B200_ERR_CUDA, "cudaStreamIsCapturing failed: %s", cudaGetErrorString(e));
    if(capture != cudaStreamCaptureStatusNone) {
        return fail(B200_ERR_STATE, "the stream is being captured: this call copies from host memory and cannot be part of a graph");
    }

    // host-side image of the scratch contents for this call (stack only)
    unsigned int blockStart[B200_NOALLOC_MAX_GROUPS + 1];
    unsigned int maxPSM = 0, maxCS = 0;
    unsigned long long period = 1;
    blockStart[0] = 0;
    for(uint32_t i = 0; i < num_groups; i++) {
        const b200_neuron_group &g = groups[i];
        if(g.num_psm > B200_MAX_PSM || g.num_cs > B200_MAX_CS) return fail(B200_ERR_INVALID, "group %u: too many children", i);
        if(g.num_delay_slots < 2) return fail(B200_ERR_INVALID, "group %u: num_delay_slots must be at least 2", i);
        if(g.first_neuron + g.num_update > g.num_neurons) return fail(B200_ERR_INVALID, "group %u: update slice out of range", i);
        if(g.first_neuron & 31u) return fail(B200_ERR_INVALID, "group %u: first_neuron must be a multiple of 32", i);
        if(!g.spk_cnt || !g.spk) return fail(B200_ERR_INVALID, "group %u: spike arrays missing", i);
        blockStart[i + 1] = blockStart[i] + (g.num_update + NEURON_BLOCK - 1) / NEURON_BLOCK;
        maxPSM = g.num_psm > maxPSM ? g.num_psm : maxPSM;
        maxCS = g.num_cs > maxCS ? g.num_cs : maxCS;
        period = foldPeriod(period, g.num_delay_slots);
        for(unsigned int p = 0; p < g.num_psm; p++) period = foldPeriod(period, g.psm[p].max_den_delay);
        if(period > (1ull << 30)) return fail(B200_ERR_INVALID, "ring sizes have no common period below 2^30");
    }
    if(blockStart[num_groups] == 0) return B200_OK;

    unsigned char *base = nullptr;
    const int s = scratchAddress(device, &base);
    if(s) return s;
    Scratch *scratch = reinterpret_cast<Scratch*>(base);
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // Everything the kernel reads from the scratch is rewritten here, in stream
    // order, so nothing survives from an earlier call: counters and ticket
    // included.  The sources are pageable host memory, which cudaMemcpyAsync
    // stages before it returns.
    StepState state = {};
    state.timestep = timestep;
    state.steps_done = steps_done;
    state.ticket = 0;
    state.error = 0;
    state.phase = (unsigned int)(steps_done % period);
    state.ring_period = (unsigned int)period;
    e = cudaMemcpyAsync(&scratch->state, &state, sizeof(state), cudaMemcpyHostToDevice, st);
    if(e == cudaSuccess) e = cudaMemcpyAsync(scratch->blockStart, blockStart, sizeof(unsigned int) * (num_groups + 1), cudaMemcpyHostToDevice, st);
    if(e == cudaSuccess) e = cudaMemcpyAsync(scratch->groups, groups, sizeof(b200_neuron_group) * num_groups, cudaMemcpyHostToDevice, st);
    if(e != cudaSuccess) return fail(B200_ERR_CUDA, "copy into the scratch array failed: %s", cudaGetErrorString(e));

    NeuronLaunch L;
    L.groups = scratch->groups;
    L.block_start = scratch->blockStart;
    L.num_groups = num_groups;
    L.batch = batch_size;
    L.dt = (float)dt;
    L.seed = seed;
    L.num_recording_timesteps = num_recording_timesteps;
    L.state = &scratch->state;
    L.count_events = 0;
    const dim3 grid(blockStart[num_groups], batch_size, 1);
    const int P = (maxPSM <= 1) ? 1 : (maxPSM <= 2) ? 2 : B200_MAX_PSM;
    const int C = (maxCS == 0) ? 0 : (maxCS == 1) ? 1 : B200_MAX_CS;
    if(P == 1 && C == 0) launch<1, 0>(L, grid, st);
    else if(P == 1 && C == 1) launch<1, 1>(L, grid, st);
    else if(P == 1) launch<1, B200_MAX_CS>(L, grid, st);
    else if(P == 2 && C == 0) launch<2, 0>(L, grid, st);
    else if(P == 2 && C == 1) launch<2, 1>(L, grid, st);
    else if(P == 2) launch<2, B200_MAX_CS>(L, grid, st);
    else if(C == 0) launch<B200_MAX_PSM, 0>(L, grid, st);
    else if(C == 1) launch<B200_MAX_PSM, 1>(L, grid, st);
    else launch<B200_MAX_PSM, B200_MAX_CS>(L, grid, st);
    e = cudaPeekAtLastError();
    if(e != cudaSuccess) return fail(B200_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return B200_OK;
}

int b200_noalloc_check(int device, void *stream)
{
    if(device < 0 || device >= MAX_DEVICES) return fail(B200_ERR_INVALID, "device index %d out of range", device);
    DeviceGuard guard;
    cudaError_t e = guard.enter(device);
    if(e != cudaSuccess) return fail(B200_ERR_CUDA, "cudaSetDevice(%d) failed: %s", device, cudaGetErrorString(e));
    unsigned char *base = nullptr;
    const int s = scratchAddress(device, &base);
    if(s) return s;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int word = 0;      // on the stack: nothing is allocated
    e = cudaMemcpyAsync(&word, &reinterpret_cast<Scratch*>(base)->state.error, sizeof(word), cudaMemcpyDeviceToHost, st);
    if(e == cudaSuccess) e = cudaStreamSynchronize(st);
    if(e != cudaSuccess) return fail(B200_ERR_CUDA, "reading the check word failed: %s", cudaGetErrorString(e));
    if(word) {
        return fail(B200_ERR_DEVICE_CHECK, "device-side check failed (0x%x):%s%s%s", word,
                    (word & ERR_SPIKE_OVERFLOW) ? " more spikes in a step than the spike list holds" : "",
                    (word & ERR_IND_RANGE) ? " index out of range" : "",
                    (word & ERR_DELAY_RANGE) ? " delay out of range" : "");
    }
    return B200_OK;
}

}   // extern "C"
