// B200 code-generation backend: implementation.  See backend.h for the design.
//
// Reference counterparts, by function (paths relative to the GeNN 5.4.0 tree):
//   genNeuronUpdate    backendSIMT.cc:320-662 + backendCUDAHIP.cc:306-449
//   genSynapseUpdate   backendSIMT.cc:664-866, presynapticUpdateStrategySIMT.cc, backendCUDAHIP.cc:451-621
//   genCustomUpdate    backendSIMT.cc:868-1154, backendCUDAHIP.cc:623-884
//   genInit            backendSIMT.cc:1368-1779, backendCUDAHIP.cc:886-1071
//   Array, State       src/genn/backends/cuda/backend.cc:73-259
// The per-group model code (sim code, threshold, reset, postsynaptic and weight-update
// snippets, initialisation snippets) is emitted by GeNN's own group classes, called back
// from here exactly as every GeNN backend does; the kernel scaffolds around it are this
// file's own.
#include "backend.h"

#include <algorithm>
#include <cassert>
#include <cstring>
#include <numeric>
#include <sstream>

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <plog/Log.h>

#include "gennUtils.h"
#include "logging.h"
#include "type.h"
#include "code_generator/codeGenUtils.h"
#include "code_generator/codeStream.h"
#include "code_generator/customUpdateGroupMerged.h"
#include "code_generator/initGroupMerged.h"
#include "code_generator/modelSpecMerged.h"
#include "code_generator/neuronUpdateGroupMerged.h"
#include "code_generator/standardLibrary.h"
#include "code_generator/synapseUpdateGroupMerged.h"

using namespace GeNN;
using namespace GeNN::CodeGenerator;

namespace
{
#define B200_CHECK_CUDA(call)                                                                               \
    do {                                                                                                    \
        const cudaError_t b200Error = (call);                                                               \
        if(b200Error != cudaSuccess) {                                                                      \
            throw std::runtime_error(std::string(__FILE__) + ": " + std::to_string(__LINE__) +              \
                                     ": cuda error " + std::to_string((int)b200Error) + ": " +              \
                                     cudaGetErrorString(b200Error));                                        \
        }                                                                                                   \
    } while(0)

// Random number functions of the model code (gennrand_*): the per-thread generator `_rng` is a
// counter-based Philox stream created in the kernel prologue (genn_b200_gen.cuh); it has no state
// in memory.
const EnvironmentLibrary::Library floatRandomFunctions = {
    {"gennrand", {Type::ResolvedType::createFunction(Type::Uint32, {}), "b200gen::u32($(_rng))"}},
    {"gennrand_uniform", {Type::ResolvedType::createFunction(Type::Float, {}), "b200gen::uniform($(_rng))"}},
    {"gennrand_normal", {Type::ResolvedType::createFunction(Type::Float, {}), "b200gen::normal($(_rng))"}},
    {"gennrand_exponential", {Type::ResolvedType::createFunction(Type::Float, {}), "b200gen::exponential($(_rng))"}},
    {"gennrand_log_normal", {Type::ResolvedType::createFunction(Type::Float, {Type::Float, Type::Float}), "b200gen::logNormal($(_rng), $(0), $(1))"}},
    {"gennrand_gamma", {Type::ResolvedType::createFunction(Type::Float, {Type::Float}), "b200gen::gamma($(_rng), $(0))"}},
    {"gennrand_binomial", {Type::ResolvedType::createFunction(Type::Uint32, {Type::Uint32, Type::Float}), "b200gen::binomial($(_rng), $(0), $(1))"}},
};
const EnvironmentLibrary::Library doubleRandomFunctions = {
    {"gennrand", {Type::ResolvedType::createFunction(Type::Uint32, {}), "b200gen::u32($(_rng))"}},
    {"gennrand_uniform", {Type::ResolvedType::createFunction(Type::Double, {}), "(double)b200gen::uniform($(_rng))"}},
    {"gennrand_normal", {Type::ResolvedType::createFunction(Type::Double, {}), "(double)b200gen::normal($(_rng))"}},
    {"gennrand_exponential", {Type::ResolvedType::createFunction(Type::Double, {}), "(double)b200gen::exponential($(_rng))"}},
    {"gennrand_log_normal", {Type::ResolvedType::createFunction(Type::Double, {Type::Double, Type::Double}), "(double)b200gen::logNormal($(_rng), (float)$(0), (float)$(1))"}},
    {"gennrand_gamma", {Type::ResolvedType::createFunction(Type::Double, {Type::Double}), "(double)b200gen::gamma($(_rng), (float)$(0))"}},
    {"gennrand_binomial", {Type::ResolvedType::createFunction(Type::Uint32, {Type::Uint32, Type::Double}), "b200gen::binomial($(_rng), $(0), (float)$(1))"}},
};

const EnvironmentLibrary::Library &randomFunctions(const Type::ResolvedType &precision)
{
    return (precision == Type::Float) ? floatRandomFunctions : doubleRandomFunctions;
}

// device functions the backend adds to every kernel environment
const EnvironmentLibrary::Library backendFunctions = {
    {"clz", {Type::ResolvedType::createFunction(Type::Int32, {Type::Uint32}), "__clz($(0))"}},
    {"atomic_or", {Type::ResolvedType::createFunction(Type::Void, {Type::Uint32.createPointer(), Type::Uint32}), "atomicOr($(0), $(1))"}},
};

size_t padTo(size_t n, size_t multiple)
{
    return ((n + multiple - 1) / multiple) * multiple;
}

//! Distinguishes the random streams of the kernels of one model: every merged group of every
//! kernel kind gets its own stream id
enum StreamKind : unsigned int
{
    STREAM_NEURON = 0x10000u, STREAM_PRESYNAPTIC = 0x20000u, STREAM_POSTSYNAPTIC = 0x30000u, STREAM_DYNAMICS = 0x40000u,
    STREAM_CUSTOM = 0x50000u, STREAM_CUSTOM_WU = 0x60000u, STREAM_INIT_NEURON = 0x70000u, STREAM_INIT_SYNAPSE = 0x80000u,
    STREAM_INIT_CONNECT = 0x90000u, STREAM_INIT_SPARSE = 0xA0000u, STREAM_INIT_CUSTOM = 0xB0000u,
    STREAM_INIT_CUSTOM_WU = 0xC0000u, STREAM_INIT_CUSTOM_WU_SPARSE = 0xD0000u, STREAM_PROCEDURAL = 0xE0000u,
    // (the group index occupies the bits from 20 up: everything here stays below 1 << 20)
    STREAM_INIT_CCU_PRE = 0xF0000u, STREAM_INIT_CCU_POST = 0xF4000u, STREAM_INIT_CCU_SPARSE = 0xF8000u, STREAM_CCU = 0xFC000u
};

//! One generated kernel of one merged group: its start-id table and launch geometry
struct KernelLaunch
{
    std::string name;           // kernel name
    size_t numThreads = 0;      // padded total over the groups
    bool batched = false;       // grid.y = batch size
};

//! Emits `__device__ unsigned int <name>[] = {...};` with the first thread id of every group
template<typename G, typename S>
size_t genStartIDs(CodeStream &os, const std::string &name, const G &mergedGroup, size_t block, S getNumThreads)
{
    os << "__device__ unsigned int " << name << "[] = {";
    size_t id = 0;
    for(const auto &g : mergedGroup.getGroups()) {
        os << id << ", ";
        id += padTo(std::max<size_t>(1, getNumThreads(g.get())), block);
    }
    os << id << "};" << std::endl;
    return id;
}

//! Kernel prologue: global thread id, the group this thread serves and its id inside the group
void genFindGroup(CodeStream &os, const std::string &structName, const std::string &arrayName, const std::string &startName,
                  size_t numGroups)
{
    os << "const unsigned int b200Thread = (blockIdx.x * blockDim.x) + threadIdx.x;" << std::endl;
    if(numGroups == 1) {
        os << "const " << structName << " *group = &" << arrayName << "[0];" << std::endl;
        os << "const unsigned int b200Group = 0;" << std::endl;
        os << "const unsigned int b200Local = b200Thread;" << std::endl;
    }
    else {
        os << "unsigned int b200Lo = 0, b200Hi = " << numGroups << ";" << std::endl;
        os << "while((b200Hi - b200Lo) > 1)";
        {
            CodeStream::Scope b(os);
            os << "const unsigned int b200Mid = (b200Lo + b200Hi) / 2;" << std::endl;
            os << "if(b200Thread >= " << startName << "[b200Mid]) b200Lo = b200Mid; else b200Hi = b200Mid;" << std::endl;
        }
        os << "const " << structName << " *group = &" << arrayName << "[b200Lo];" << std::endl;
        os << "const unsigned int b200Group = b200Lo;" << std::endl;
        os << "const unsigned int b200Local = b200Thread - " << startName << "[b200Lo];" << std::endl;
    }
}

//! `__device__` array of merged-group structs plus the push function the runtime calls through
//! libffi (runtime.h:573-669); fields in the order GroupMerged::getSortedFields gives
template<typename T>
void genDeviceStructArrayPush(CodeStream &os, const BackendBase &backend, const std::vector<T> &groups)
{
    for(const auto &g : groups) {
        const std::string structName = "Merged" + T::name + "Group" + std::to_string(g.getIndex());
        os << "__device__ " << structName << " d_merged" << T::name << "Group" << g.getIndex() << "[" << g.getGroups().size() << "];" << std::endl;
        if(g.getFields().empty()) {
            continue;
        }
        os << "void pushMerged" << T::name << "Group" << g.getIndex() << "ToDevice(unsigned int idx, ";
        g.generateStructFieldArgumentDefinitions(os, backend);
        os << ")";
        {
            CodeStream::Scope b(os);
            os << structName << " group = {";
            for(const auto &f : g.getSortedFields(backend)) {
                os << f.name << ", ";
            }
            os << "};" << std::endl;
            os << "CHECK_RUNTIME_ERRORS(cudaMemcpyToSymbolAsync(d_merged" << T::name << "Group" << g.getIndex() << ", &group, sizeof(" << structName << "), ";
            os << "idx * sizeof(" << structName << "), cudaMemcpyHostToDevice, 0));" << std::endl;
        }
    }
}

//! Merged groups whose code runs on the host: the array of group structures lives in host memory
template<typename T>
void genHostStructArrayPush(CodeStream &os, const BackendBase &backend, const std::vector<T> &groups)
{
    for(const auto &g : groups) {
        const std::string structName = "Merged" + T::name + "Group" + std::to_string(g.getIndex());
        os << "static " << structName << " merged" << T::name << "Group" << g.getIndex() << "[" << g.getGroups().size() << "];" << std::endl;
        if(g.getFields().empty()) {
            continue;
        }
        os << "void pushMerged" << T::name << "Group" << g.getIndex() << "ToDevice(unsigned int idx, ";
        g.generateStructFieldArgumentDefinitions(os, backend);
        os << ")";
        {
            CodeStream::Scope b(os);
            for(const auto &f : g.getSortedFields(backend)) {
                os << "merged" << T::name << "Group" << g.getIndex() << "[idx]." << f.name << " = " << f.name << ";" << std::endl;
            }
        }
    }
}

//! Host-side launch of a generated kernel on stream 0
void genLaunch(CodeStream &os, const KernelLaunch &k, size_t block, unsigned int batchSize, const std::string &args)
{
    if(k.numThreads == 0) {
        return;
    }
    CodeStream::Scope b(os);
    os << "const dim3 threads(" << block << ", 1);" << std::endl;
    os << "const dim3 grid(" << (k.numThreads / block) << ", " << (k.batched ? batchSize : 1u) << ");" << std::endl;
    os << k.name << "<<<grid, threads>>>(" << args << ");" << std::endl;
    os << "CHECK_RUNTIME_ERRORS(cudaPeekAtLastError());" << std::endl;
}

void genKernelTimerStart(CodeStream &os, const std::string &name, bool enabled)
{
    if(enabled) {
        os << "CHECK_RUNTIME_ERRORS(cudaEventRecord(" << name << "Start));" << std::endl;
    }
}

void genKernelTimerStop(CodeStream &os, const std::string &name, bool enabled, bool readBack)
{
    if(enabled) {
        os << "CHECK_RUNTIME_ERRORS(cudaEventRecord(" << name << "Stop));" << std::endl;
        if(readBack) {
            CodeStream::Scope b(os);
            os << "CHECK_RUNTIME_ERRORS(cudaEventSynchronize(" << name << "Stop));" << std::endl;
            os << "float b200Elapsed;" << std::endl;
            os << "CHECK_RUNTIME_ERRORS(cudaEventElapsedTime(&b200Elapsed, " << name << "Start, " << name << "Stop));" << std::endl;
            os << name << "Time += b200Elapsed / 1000.0;" << std::endl;
        }
    }
}
}   // anonymous namespace

namespace GeNN::CodeGenerator::B200
{
//--------------------------------------------------------------------------
// Preferences
//--------------------------------------------------------------------------
void Preferences::updateHash(boost::uuids::detail::sha1 &hash) const
{
    PreferencesBase::updateHash(hash);
    Utils::updateHash(deviceID, hash);
    Utils::updateHash(blockSize, hash);
}

//--------------------------------------------------------------------------
// Array
//--------------------------------------------------------------------------
Array::Array(const Type::ResolvedType &type, size_t count, VarLocation location, bool uninitialized)
:   Runtime::ArrayBase(type, count, location, uninitialized)
{
    if(count > 0) {
        allocate(count);
    }
}

Array::~Array()
{
    if(getCount() > 0) {
        free();
    }
}

void Array::allocate(size_t count)
{
    setCount(count);
    // the runtime wraps the host pointer in views for every location with a host side
    // (pygenn/src/runtime.cc:31-36); page-locked so that pushes and pulls run at link speed
    if(getLocation() & VarLocationAttribute::HOST) {
        std::byte *host = nullptr;
        B200_CHECK_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&host), getSizeBytes(), cudaHostAllocPortable));
        setHostPointer(host);
    }
    if(getLocation() & VarLocationAttribute::DEVICE) {
        // 256 bytes of slack: kernels may read whole vectors that straddle the end of an unaligned row
        B200_CHECK_CUDA(cudaMalloc(reinterpret_cast<void**>(&m_DevicePointer), getSizeBytes() + 256));
    }
}

void Array::free()
{
    if(getHostPointer()) {
        B200_CHECK_CUDA(cudaFreeHost(getHostPointer()));
        setHostPointer(nullptr);
    }
    if(m_DevicePointer) {
        B200_CHECK_CUDA(cudaFree(m_DevicePointer));
        m_DevicePointer = nullptr;
    }
    setCount(0);
}

void Array::pushToDevice()
{
    if(!(getLocation() & VarLocationAttribute::HOST) || !(getLocation() & VarLocationAttribute::DEVICE)) {
        throw std::runtime_error("Cannot push array that isn't present on host and device");
    }
    B200_CHECK_CUDA(cudaMemcpy(m_DevicePointer, getHostPointer(), getSizeBytes(), cudaMemcpyHostToDevice));
}

void Array::pullFromDevice()
{
    if(!(getLocation() & VarLocationAttribute::HOST) || !(getLocation() & VarLocationAttribute::DEVICE)) {
        throw std::runtime_error("Cannot pull array that isn't present on host and device");
    }
    B200_CHECK_CUDA(cudaMemcpy(getHostPointer(), m_DevicePointer, getSizeBytes(), cudaMemcpyDeviceToHost));
}

void Array::pushSlice1DToDevice(size_t offset, size_t count)
{
    if(offset + count > getCount()) {
        throw std::runtime_error("Cannot push slice that overflows array");
    }
    const size_t bytes = getType().getValue().size;
    B200_CHECK_CUDA(cudaMemcpy(m_DevicePointer + (offset * bytes), getHostPointer() + (offset * bytes), count * bytes, cudaMemcpyHostToDevice));
}

void Array::pullSlice1DFromDevice(size_t offset, size_t count)
{
    if(offset + count > getCount()) {
        throw std::runtime_error("Cannot pull slice that overflows array");
    }
    const size_t bytes = getType().getValue().size;
    B200_CHECK_CUDA(cudaMemcpy(getHostPointer() + (offset * bytes), m_DevicePointer + (offset * bytes), count * bytes, cudaMemcpyDeviceToHost));
}

void Array::memsetDeviceObject(int value)
{
    B200_CHECK_CUDA(cudaMemset(m_DevicePointer, value, getSizeBytes()));
}

void Array::serialiseDeviceObject(std::vector<std::byte> &bytes, bool pointerToPointer) const
{
    std::byte vBytes[sizeof(void*)];
    if(pointerToPointer) {
        std::byte *const *devicePointerPointer = &m_DevicePointer;
        std::memcpy(vBytes, &devicePointerPointer, sizeof(void*));
    }
    else {
        std::memcpy(vBytes, &m_DevicePointer, sizeof(void*));
    }
    std::copy(std::begin(vBytes), std::end(vBytes), std::back_inserter(bytes));
}

void Array::serialiseHostObject(std::vector<std::byte>&, bool) const
{
    throw std::runtime_error("The B200 backend has no host objects");
}

//--------------------------------------------------------------------------
// Factory
//--------------------------------------------------------------------------
Backend createBackend(const ModelSpecInternal&, const filesystem::path&, plog::Severity backendLevel,
                      plog::IAppender *backendAppender, const Preferences &preferences)
{
    if(plog::get<Logging::CHANNEL_BACKEND>() == nullptr) {
        plog::init<Logging::CHANNEL_BACKEND>(backendLevel, backendAppender);
    }
    else {
        plog::get<Logging::CHANNEL_BACKEND>()->setMaxSeverity(backendLevel);
    }
    if(preferences.blockSize == 0 || (preferences.blockSize % 32) != 0 || preferences.blockSize > 1024) {
        throw std::runtime_error("B200 backend: blockSize must be a multiple of 32 up to 1024");
    }
    return Backend(preferences);
}

//--------------------------------------------------------------------------
// Backend: construction, simple virtuals
//--------------------------------------------------------------------------
Backend::Backend(const Preferences &preferences)
:   BackendBase(preferences)
{
    setPointerBytes(sizeof(void*));
}

std::string Backend::includeDirectory() const
{
    const auto &p = getPreferences<Preferences>();
    if(!p.includePath.empty()) {
        return p.includePath;
    }
    // <repo>/genn_b200/backend/libgenn_b200_backend.so -> <repo>/include
    Dl_info info;
    if(dladdr(reinterpret_cast<const void*>(&createBackend), &info) && info.dli_fname) {
        std::string path(info.dli_fname);
        for(int up = 0; up < 3; up++) {
            const size_t slash = path.find_last_of('/');
            path = (slash == std::string::npos) ? "." : path.substr(0, slash);
        }
        return path + "/include";
    }
    return "include";
}

size_t Backend::getSynapticMatrixRowStride(const SynapseGroupInternal &sg) const
{
    // the row strides PyGeNN assumes when it fills host views (pygenn/genn_groups.py:41-48)
    if((sg.getMatrixType() & SynapseMatrixConnectivity::SPARSE) || (sg.getMatrixType() & SynapseMatrixConnectivity::TOEPLITZ)) {
        return sg.getMaxConnections();
    }
    else if(sg.getMatrixType() & SynapseMatrixConnectivity::BITMASK) {
        return padTo(sg.getTrgNeuronGroup()->getNumNeurons(), 32);
    }
    else {
        return sg.getTrgNeuronGroup()->getNumNeurons();
    }
}

void Backend::genDefinitionsPreamble(CodeStream &os, const ModelSpecMerged&) const
{
    os << "// Standard C++ includes" << std::endl;
    os << "#include <random>" << std::endl;
    os << "#include <string>" << std::endl;
    os << "#include <stdexcept>" << std::endl;
    os << std::endl;
    os << "// Standard C includes" << std::endl;
    os << "#include <cassert>" << std::endl;
    os << "#include <cmath>" << std::endl;
    os << "#include <cstdint>" << std::endl;
    os << "#include <cstring>" << std::endl;
    os << std::endl;
    os << "// CUDA" << std::endl;
    os << "#include <cuda_runtime.h>" << std::endl;
    os << std::endl;
    os << "#define CHECK_RUNTIME_ERRORS(call) {\\" << std::endl;
    os << "    cudaError_t error = call;\\" << std::endl;
    os << "    if (error != cudaSuccess) {\\" << std::endl;
    os << "        throw std::runtime_error(__FILE__\": \" + std::to_string(__LINE__) + \": cuda error \" + std::to_string(error) + \": \" + cudaGetErrorString(error));\\" << std::endl;
    os << "    }\\" << std::endl;
    os << "}" << std::endl;
    os << std::endl;
    os << "// seed of every Philox stream: the model's seed, or drawn from the system when that is zero" << std::endl;
    os << "extern unsigned long long b200Seed;" << std::endl;
    os << "// Device helpers of the B200 backend (spike compaction, Philox streams)" << std::endl;
    os << "#if defined(__CUDACC__)" << std::endl;
    os << "#include \"genn_b200_gen.cuh\"" << std::endl;
    os << "#endif" << std::endl;
    os << std::endl;
}

void Backend::genRunnerPreamble(CodeStream &os, const ModelSpecMerged&) const
{
    os << "unsigned long long b200Seed = 0;" << std::endl;
}

void Backend::genAllocateMemPreamble(CodeStream &os, const ModelSpecMerged &modelMerged) const
{
    os << "CHECK_RUNTIME_ERRORS(cudaSetDevice(" << getPreferences<Preferences>().deviceID << "));" << std::endl;
    if(modelMerged.getModel().getSeed() == 0) {
        os << "{ std::random_device b200SeedSource; b200Seed = ((unsigned long long)b200SeedSource() << 32) | b200SeedSource(); }" << std::endl;
    }
    else {
        os << "b200Seed = " << modelMerged.getModel().getSeed() << "ull;" << std::endl;
    }
}

void Backend::genFreeMemPreamble(CodeStream&, const ModelSpecMerged&) const
{
}

void Backend::genStepTimeFinalisePreamble(CodeStream &os, const ModelSpecMerged &modelMerged) const
{
    // kernel timers are read back once per step, as the reference does (backendCUDAHIP.cc:1400-1411)
    if(modelMerged.getModel().isTimingEnabled()) {
        os << "CHECK_RUNTIME_ERRORS(cudaDeviceSynchronize());" << std::endl;
    }
}

std::unique_ptr<GeNN::Runtime::StateBase> Backend::createState(const Runtime::Runtime&) const
{
    B200_CHECK_CUDA(cudaSetDevice(getPreferences<Preferences>().deviceID));
    return std::make_unique<State>();
}

std::unique_ptr<GeNN::Runtime::ArrayBase> Backend::createArray(const Type::ResolvedType &type, size_t count,
                                                               VarLocation location, bool uninitialized) const
{
    return std::make_unique<Array>(type, count, location, uninitialized);
}

std::unique_ptr<GeNN::Runtime::ArrayBase> Backend::createPopulationRNG(size_t) const
{
    // random streams are stateless (keyed on seed, group, neuron, time step): one placeholder word
    return std::make_unique<Array>(Type::Uint32, 1, VarLocation::DEVICE, false);
}

void Backend::genLazyVariableDynamicAllocation(CodeStream &os, const Type::ResolvedType &type, const std::string &name,
                                               VarLocation loc, const std::string &countVarName) const
{
    const auto &underlyingType = type.isPointer() ? *type.getPointer().valueType : type;
    const std::string hostPointer = type.isPointer() ? ("*$(_" + name + ")") : ("$(_" + name + ")");
    const std::string hostPointerToPointer = type.isPointer() ? ("$(_" + name + ")") : ("&$(_" + name + ")");
    const std::string devicePointerToPointer = type.isPointer() ? ("$(_d_" + name + ")") : ("&$(_d_" + name + ")");
    if(loc & VarLocationAttribute::HOST) {
        os << "CHECK_RUNTIME_ERRORS(cudaHostAlloc(" << hostPointerToPointer << ", " << countVarName << " * sizeof(" << underlyingType.getName() << "), cudaHostAllocPortable));" << std::endl;
    }
    if(loc & VarLocationAttribute::DEVICE) {
        os << "CHECK_RUNTIME_ERRORS(cudaMalloc(" << devicePointerToPointer << ", " << countVarName << " * sizeof(" << underlyingType.getName() << ")));" << std::endl;
    }
    (void)hostPointer;
}

void Backend::genLazyVariableDynamicPush(CodeStream &os, const Type::ResolvedType &type, const std::string &name,
                                         VarLocation loc, const std::string &countVarName) const
{
    if(loc & VarLocationAttribute::HOST) {
        if(type.isPointer()) {
            os << "CHECK_RUNTIME_ERRORS(cudaMemcpy(*$(_d_" << name << "), *$(_" << name << "), ";
            os << countVarName << " * sizeof(" << type.getPointer().valueType->getName() << "), cudaMemcpyHostToDevice));" << std::endl;
        }
        else {
            os << "CHECK_RUNTIME_ERRORS(cudaMemcpy($(_d_" << name << "), $(_" << name << "), ";
            os << countVarName << " * sizeof(" << type.getName() << "), cudaMemcpyHostToDevice));" << std::endl;
        }
    }
}

void Backend::genLazyVariableDynamicPull(CodeStream &os, const Type::ResolvedType &type, const std::string &name,
                                         VarLocation loc, const std::string &countVarName) const
{
    if(loc & VarLocationAttribute::HOST) {
        if(type.isPointer()) {
            os << "CHECK_RUNTIME_ERRORS(cudaMemcpy(*$(_" << name << "), *$(_d_" << name << "), ";
            os << countVarName << " * sizeof(" << type.getPointer().valueType->getName() << "), cudaMemcpyDeviceToHost));" << std::endl;
        }
        else {
            os << "CHECK_RUNTIME_ERRORS(cudaMemcpy($(_" << name << "), $(_d_" << name << "), ";
            os << countVarName << " * sizeof(" << type.getName() << "), cudaMemcpyDeviceToHost));" << std::endl;
        }
    }
}

void Backend::genMergedDynamicVariablePush(CodeStream &os, const std::string &suffix, size_t mergedGroupIdx,
                                           const std::string &groupIdx, const std::string &fieldName,
                                           const std::string &egpName) const
{
    const std::string structName = "Merged" + suffix + "Group" + std::to_string(mergedGroupIdx);
    os << "CHECK_RUNTIME_ERRORS(cudaMemcpyToSymbolAsync(d_merged" << suffix << "Group" << mergedGroupIdx;
    os << ", &" << egpName << ", sizeof(" << egpName << ")";
    os << ", (sizeof(" << structName << ") * (" << groupIdx << ")) + offsetof(" << structName << ", " << fieldName << ")";
    os << ", cudaMemcpyHostToDevice, 0));" << std::endl;
}

std::string Backend::getAtomicOperation(const std::string &lhsPointer, const std::string &rhsValue,
                                        const Type::ResolvedType &type, AtomicOperation op) const
{
    if(op == AtomicOperation::ADD) {
        return "atomicAdd(" + lhsPointer + ", " + rhsValue + ")";
    }
    else {
        assert(op == AtomicOperation::OR);
        assert(type == Type::Uint32 || type == Type::Int32);
        return "atomicOr(" + lhsPointer + ", " + rhsValue + ")";
    }
}

void Backend::genGlobalDeviceRNG(CodeStream&, CodeStream&, CodeStream&, CodeStream&) const
{
    // no global generator object: every thread derives its Philox stream from the model seed
}

void Backend::genTimer(CodeStream &definitions, CodeStream &runner, CodeStream &allocations, CodeStream &free,
                       CodeStream&, const std::string &name, bool) const
{
    definitions << "extern cudaEvent_t " << name << "Start;" << std::endl;
    definitions << "extern cudaEvent_t " << name << "Stop;" << std::endl;
    runner << "cudaEvent_t " << name << "Start;" << std::endl;
    runner << "cudaEvent_t " << name << "Stop;" << std::endl;
    allocations << "CHECK_RUNTIME_ERRORS(cudaEventCreate(&" << name << "Start));" << std::endl;
    allocations << "CHECK_RUNTIME_ERRORS(cudaEventCreate(&" << name << "Stop));" << std::endl;
    free << "CHECK_RUNTIME_ERRORS(cudaEventDestroy(" << name << "Start));" << std::endl;
    free << "CHECK_RUNTIME_ERRORS(cudaEventDestroy(" << name << "Stop));" << std::endl;
}

void Backend::genReturnFreeDeviceMemoryBytes(CodeStream &os) const
{
    os << "size_t free; size_t total;" << std::endl;
    os << "CHECK_RUNTIME_ERRORS(cudaMemGetInfo(&free, &total));" << std::endl;
    os << "return free;" << std::endl;
}

void Backend::genAssert(CodeStream &os, const std::string &condition) const
{
    os << "assert(" << condition << ");" << std::endl;
}

//--------------------------------------------------------------------------
// Build rules: every module is CUDA, compiled for sm_100a only
//--------------------------------------------------------------------------
void Backend::genMakefilePreamble(std::ostream &os) const
{
    const auto &p = getPreferences<Preferences>();
    std::string flags = "-gencode arch=compute_100a,code=sm_100a -std=c++17 -x cu -Xcompiler -fPIC -lineinfo";
    flags += " -diag-suppress 177,550 -I\"" + includeDirectory() + "\"";
    flags += p.debugCode ? " -O0 -g -G" : " -O3";
    if(p.optimizeCode) {
        flags += " -use_fast_math";
    }
    else {
        // model arithmetic is compared with the CPU backend: no contraction into fused multiply-adds
        flags += " -fmad=false";
    }
    flags += " " + p.userNvccFlagsGNU;
    os << "NVCC := " << p.nvccPath << std::endl;
    os << "NVCCFLAGS := " << flags << std::endl;
    os << "LINKFLAGS := -gencode arch=compute_100a,code=sm_100a --shared -Xcompiler -fPIC" << std::endl;
    os << std::endl;
}

void Backend::genMakefileLinkRule(std::ostream &os) const
{
    os << "\t@$(NVCC) $(LINKFLAGS) -o $@ $(OBJECTS)" << std::endl;
}

void Backend::genMakefileCompileRule(std::ostream &os) const
{
    os << "%.d: ;" << std::endl;
    os << "%.o: %.cc %.d" << std::endl;
    os << "\t@$(NVCC) -c $(NVCCFLAGS) -o $@ $<" << std::endl;
}

void Backend::genNMakefilePreamble(std::ostream&) const { assert(false); }
void Backend::genNMakefileLinkRule(std::ostream&) const { assert(false); }
void Backend::genNMakefileCompileRule(std::ostream&) const { assert(false); }
void Backend::genMSBuildConfigProperties(std::ostream&) const { assert(false); }
void Backend::genMSBuildImportProps(std::ostream&) const { assert(false); }
void Backend::genMSBuildItemDefinitions(std::ostream&) const { assert(false); }
void Backend::genMSBuildCompileModule(const std::string&, std::ostream&) const { assert(false); }
void Backend::genMSBuildImportTarget(std::ostream&) const { assert(false); }

bool Backend::isGlobalHostRNGRequired(const ModelSpecInternal &model) const
{
    // host-side connectivity initialisation snippets draw from the host generator
    if(std::any_of(model.getSynapseGroups().cbegin(), model.getSynapseGroups().cend(),
                   [](const ModelSpec::SynapseGroupValueType &s)
                   {
                       return s.second.getSparseConnectivityInitialiser().isHostRNGRequired();
                   }))
    {
        return true;
    }
    // ... and so does the host update code of custom connectivity updates
    return std::any_of(model.getCustomConnectivityUpdates().cbegin(), model.getCustomConnectivityUpdates().cend(),
                       [](const ModelSpec::CustomConnectivityUpdateValueType &c)
                       {
                           return Utils::isRNGRequired(c.second.getHostUpdateCodeTokens());
                       });
}

bool Backend::isGlobalDeviceRNGRequired(const ModelSpecInternal&) const
{
    return false;
}

size_t Backend::getDeviceMemoryBytes() const
{
    size_t free = 0, total = 0;
    if(cudaMemGetInfo(&free, &total) != cudaSuccess) {
        return 0;
    }
    return total;
}

Backend::MemorySpaces Backend::getMergedGroupMemorySpaces(const ModelSpecMerged&) const
{
    // merged-group arrays live in __device__ memory (L2-resident and read through the
    // read-only path); there is no small memory space to ration
    return {};
}

boost::uuids::detail::sha1::digest_type Backend::getHashDigest() const
{
    boost::uuids::detail::sha1 hash;
    Utils::updateHash("B200", hash);
    getPreferences<Preferences>().updateHash(hash);
    return hash.get_digest();
}

//--------------------------------------------------------------------------
// Neuron update
//--------------------------------------------------------------------------
void Backend::genNeuronUpdate(CodeStream &os, FileStreamCreator, ModelSpecMerged &modelMerged,
                              BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const
{
    const ModelSpecInternal &model = modelMerged.getModel();
    const unsigned int batchSize = model.getBatchSize();
    const size_t block = blockSize();
    const std::string timeType = model.getTimePrecision().getName();
    const std::string dtLiteral = Type::writeNumeric(model.getDT(), model.getTimePrecision());
    const std::string kernelArgs = timeType + " t, unsigned int recordingTimestep, unsigned long long b200Step, unsigned long long b200Seed";

    std::ostringstream kernelStream;
    CodeStream kernels(kernelStream);
    std::vector<KernelLaunch> prevLaunches, queueLaunches, neuronLaunches;

    EnvironmentLibrary backendEnv(kernels, backendFunctions);
    EnvironmentLibrary mathsEnv(backendEnv, StandardLibrary::getMathsFunctions());
    EnvironmentLibrary kernelLibEnv(mathsEnv, randomFunctions(model.getPrecision()));

    // opens a kernel: signature, the names every group emitter expects, the thread's group
    auto beginKernel = [&](EnvironmentExternal &env, const std::string &structName, const std::string &arrayName,
                           const std::string &startName, size_t numGroups)
    {
        env.getStream() << "const unsigned int batch = blockIdx.y;" << std::endl;
        env.add(model.getTimePrecision().addConst(), "t", "t");
        env.add(Type::Uint32.addConst(), "batch", "batch");
        env.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
        genFindGroup(env.getStream(), structName, arrayName, startName, numGroups);
        env.add(Type::Uint32.addConst(), "id", "b200Local");
    };

    // ---- previous spike times: one thread per neuron, set prevST of last step's spikes -----------------
    modelMerged.genMergedNeuronPrevSpikeTimeUpdateGroups(
        *this, memorySpaces,
        [&](auto &n)
        {
            const std::string idx = std::to_string(n.getIndex());
            KernelLaunch launch;
            launch.name = "neuronPrevSpikeTimeUpdateKernel" + idx;
            launch.batched = true;
            launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedNeuronPrevSpikeTimeUpdateGroupStartID" + idx, n, block,
                                            [](const NeuronGroupInternal &ng){ return ng.getNumNeurons(); });
            kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
            {
                CodeStream::Scope b(kernelLibEnv.getStream());
                EnvironmentExternal kernelEnv(kernelLibEnv);
                beginKernel(kernelEnv, "MergedNeuronPrevSpikeTimeUpdateGroup" + idx, "d_mergedNeuronPrevSpikeTimeUpdateGroup" + idx,
                            "d_mergedNeuronPrevSpikeTimeUpdateGroupStartID" + idx, n.getGroups().size());
                EnvironmentGroupMergedField<NeuronPrevSpikeTimeUpdateGroupMerged> groupEnv(kernelEnv, n);
                buildStandardEnvironment(groupEnv, batchSize);
                if(n.getArchetype().isDelayRequired()) {
                    // the queue pointer still points at the slot written last step
                    if(batchSize == 1) {
                        groupEnv.printLine("const unsigned int lastTimestepDelaySlot = *$(_spk_que_ptr);");
                    }
                    else {
                        groupEnv.printLine("const unsigned int lastTimestepDelaySlot = *$(_spk_que_ptr) + ($(batch) * " + std::to_string(n.getArchetype().getNumDelaySlots()) + ");");
                    }
                    groupEnv.printLine("const unsigned int lastTimestepDelayOffset = lastTimestepDelaySlot * $(num_neurons);");
                }
                auto genUpdate = [&](EnvironmentExternalBase &env, bool trueSpike)
                {
                    const std::string suffix = trueSpike ? "" : "_event";
                    const std::string time = trueSpike ? "st" : "set";
                    const bool delay = trueSpike ? n.getArchetype().isSpikeDelayRequired() : n.getArchetype().isSpikeEventDelayRequired();
                    if(delay) {
                        env.print("if($(id) < $(_spk_cnt" + suffix + ")[lastTimestepDelaySlot])");
                        {
                            CodeStream::Scope b(env.getStream());
                            env.printLine("$(_prev_" + time + ")[lastTimestepDelayOffset + $(_spk" + suffix + ")[lastTimestepDelayOffset + $(id)]] = $(t) - $(dt);");
                        }
                    }
                    else {
                        env.print("if($(id) < $(_spk_cnt" + suffix + ")[$(batch)])");
                        {
                            CodeStream::Scope b(env.getStream());
                            if(batchSize == 1) {
                                env.printLine("$(_prev_" + time + ")[$(_spk" + suffix + ")[$(id)]] = $(t) - $(dt);");
                            }
                            else {
                                env.printLine("$(_prev_" + time + ")[$(_batch_offset) + $(_spk" + suffix + ")[$(_batch_offset) + $(id)]] = $(t) - $(dt);");
                            }
                        }
                    }
                };
                if(n.getArchetype().isPrevSpikeTimeRequired()) {
                    n.generateSpikes(groupEnv, [&](EnvironmentExternalBase &env){ genUpdate(env, true); });
                }
                if(n.getArchetype().isPrevSpikeEventTimeRequired()) {
                    n.generateSpikeEvents(groupEnv, [&](EnvironmentExternalBase &env){ genUpdate(env, false); });
                }
            }
            prevLaunches.push_back(launch);
        });

    // ---- spike queue update: one thread per group advances the queue pointer and clears the counts ----
    modelMerged.genMergedNeuronSpikeQueueUpdateGroups(
        *this, memorySpaces,
        [&](auto &n)
        {
            const std::string idx = std::to_string(n.getIndex());
            KernelLaunch launch;
            launch.name = "neuronSpikeQueueUpdateKernel" + idx;
            launch.numThreads = padTo(n.getGroups().size(), 32);
            kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "()";
            {
                CodeStream::Scope b(kernelLibEnv.getStream());
                kernelLibEnv.getStream() << "const unsigned int b200Thread = (blockIdx.x * blockDim.x) + threadIdx.x;" << std::endl;
                kernelLibEnv.getStream() << "if(b200Thread < " << n.getGroups().size() << ")";
                {
                    CodeStream::Scope b(kernelLibEnv.getStream());
                    EnvironmentExternal kernelEnv(kernelLibEnv);
                    kernelEnv.getStream() << "const MergedNeuronSpikeQueueUpdateGroup" << idx << " *group = &d_mergedNeuronSpikeQueueUpdateGroup" << idx << "[b200Thread];" << std::endl;
                    EnvironmentGroupMergedField<NeuronSpikeQueueUpdateGroupMerged> groupEnv(kernelEnv, n);
                    buildStandardEnvironment(groupEnv, batchSize);
                    n.genSpikeQueueUpdate(groupEnv, batchSize);
                }
            }
            queueLaunches.push_back(launch);
        });

    // ---- neuron update ------------------------------------------------------------------------------------------
    modelMerged.genMergedNeuronUpdateGroups(
        *this, memorySpaces,
        [&](auto &n)
        {
            const std::string idx = std::to_string(n.getIndex());
            KernelLaunch launch;
            launch.name = "updateNeuronsKernel" + idx;
            launch.batched = true;
            launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedNeuronUpdateGroupStartID" + idx, n, block,
                                            [](const NeuronGroupInternal &ng){ return ng.getNumNeurons(); });
            const size_t numEventGroups = n.getMergedSpikeEventGroups().size();
            kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
            {
                CodeStream::Scope b(kernelLibEnv.getStream());
                EnvironmentExternal kernelEnv(kernelLibEnv);
                beginKernel(kernelEnv, "MergedNeuronUpdateGroup" + idx, "d_mergedNeuronUpdateGroup" + idx,
                            "d_mergedNeuronUpdateGroupStartID" + idx, n.getGroups().size());
                EnvironmentGroupMergedField<NeuronUpdateGroupMerged> groupEnv(kernelEnv, n);
                buildStandardEnvironment(groupEnv, batchSize);

                // whether this thread's neuron emitted a spike / each kind of spike-like event this step
                groupEnv.getStream() << "bool b200Spiked = false;" << std::endl;
                for(size_t e = 0; e < numEventGroups; e++) {
                    groupEnv.getStream() << "bool b200Event" << e << " = false;" << std::endl;
                }
                groupEnv.print("if($(id) < $(num_neurons))");
                {
                    CodeStream::Scope b(groupEnv.getStream());
                    EnvironmentGroupMergedField<NeuronUpdateGroupMerged> validEnv(groupEnv, n);
                    // stateless Philox stream of (group, neuron, batch element, time step); only created if the model draws
                    validEnv.add(Type::Void, "_rng", "b200Rng",
                                 {validEnv.addInitialiser("b200gen::Rng b200Rng = b200gen::simRng(b200Seed, " + std::to_string(STREAM_NEURON + n.getIndex()) +
                                                          "u + (b200Group << 20), $(id), $(batch), b200Step);")});
                    n.generateNeuronUpdate(
                        validEnv, batchSize,
                        // true spike: flag it; everything tied to the spiking neuron's state happens here
                        [&n, batchSize](EnvironmentExternalBase &env)
                        {
                            env.printLine("b200Spiked = true;");
                            n.generateWUVarUpdate(env, batchSize);
                            if(n.getArchetype().isSpikeTimeRequired()) {
                                env.printLine("$(_st)[" + n.getWriteVarIndex(n.getArchetype().isSpikeDelayRequired(), batchSize,
                                                                            VarAccessDim::BATCH | VarAccessDim::ELEMENT, "$(id)") + "] = $(t);");
                            }
                        },
                        // spike-like event
                        [&n, batchSize](EnvironmentExternalBase &env, NeuronUpdateGroupMerged::SynSpikeEvent &sg)
                        {
                            env.printLine("b200Event" + std::to_string(sg.getIndex()) + " = true;");
                            if(n.getArchetype().isSpikeEventTimeRequired()) {
                                env.printLine("$(_set)[" + n.getWriteVarIndex(n.getArchetype().isSpikeEventDelayRequired(), batchSize,
                                                                             VarAccessDim::BATCH | VarAccessDim::ELEMENT, "$(id)") + "] = $(t);");
                            }
                        });
                }

                // all lanes of the warp are back together: compact the warp's events into the lists
                // (one atomic per warp that has any; ids ascend within a warp)
                auto genCompaction = [&](EnvironmentExternalBase &env, const std::string &flag, bool trueSpike)
                {
                    const std::string suffix = trueSpike ? "" : "_event";
                    const bool delay = trueSpike ? n.getArchetype().isSpikeDelayRequired() : n.getArchetype().isSpikeEventDelayRequired();
                    std::string countIndex;
                    if(delay) {
                        countIndex = "*$(_spk_que_ptr)";
                        if(batchSize > 1) {
                            countIndex += " + ($(batch) * " + std::to_string(n.getArchetype().getNumDelaySlots()) + ")";
                        }
                    }
                    else {
                        countIndex = "$(batch)";
                    }
                    const std::string listOffset = n.getWriteVarIndex(delay, batchSize, VarAccessDim::BATCH | VarAccessDim::ELEMENT, "");
                    env.printLine("b200gen::emitEvents(" + flag + ", $(id), &$(_spk_cnt" + suffix + ")[" + countIndex + "], &$(_spk" + suffix + ")[" + listOffset + "0]);");
                };
                const bool emitsSpikes = n.getArchetype().isTrueSpikeRequired() || !n.getMergedSpikeGroups().empty();
                if(emitsSpikes) {
                    n.generateSpikes(groupEnv, [&](EnvironmentExternalBase &env){ genCompaction(env, "b200Spiked", true); });
                }
                n.generateSpikeEvents(groupEnv,
                                      [&](EnvironmentExternalBase &env, NeuronUpdateGroupMerged::SynSpikeEvent &sg)
                                      {
                                          genCompaction(env, "b200Event" + std::to_string(sg.getIndex()), false);
                                      });

                // recording: a warp covers exactly one 32-neuron word (groups start on block boundaries)
                if(n.getArchetype().isSpikeRecordingEnabled() || n.getArchetype().isSpikeEventRecordingEnabled()) {
                    groupEnv.printLine("const unsigned int numRecordingWords = ($(num_neurons) + 31) / 32;");
                    std::string globalIndex = "(recordingTimestep * numRecordingWords * " + std::to_string(batchSize) + ") + ($(id) / 32)";
                    if(batchSize > 1) {
                        globalIndex += " + ($(batch) * numRecordingWords)";
                    }
                    if(n.getArchetype().isSpikeRecordingEnabled()) {
                        groupEnv.printLine("b200gen::recordEvents(b200Spiked, $(id), numRecordingWords, &$(_record_spk)[" + globalIndex + "]);");
                    }
                    if(n.getArchetype().isSpikeEventRecordingEnabled()) {
                        n.generateSpikeEvents(groupEnv,
                                              [&](EnvironmentExternalBase &env, NeuronUpdateGroupMerged::SynSpikeEvent &sg)
                                              {
                                                  env.printLine("b200gen::recordEvents(b200Event" + std::to_string(sg.getIndex()) + ", $(id), numRecordingWords, &$(_record_spk_event)[" + globalIndex + "]);");
                                              });
                    }
                }
            }
            neuronLaunches.push_back(launch);
        });

    // ---- file: structs, device arrays + push functions, dynamic-field pushes, kernels, host function ----
    modelMerged.genMergedNeuronUpdateGroupStructs(os, *this);
    modelMerged.genMergedNeuronSpikeQueueUpdateStructs(os, *this);
    modelMerged.genMergedNeuronPrevSpikeTimeUpdateStructs(os, *this);
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedNeuronUpdateGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedNeuronSpikeQueueUpdateGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedNeuronPrevSpikeTimeUpdateGroups());
    preambleHandler(os);
    os << kernelStream.str();

    os << "void updateNeurons(" << timeType << " t";
    if(model.isRecordingInUse()) {
        os << ", unsigned int recordingTimestep";
    }
    os << ")";
    {
        CodeStream::Scope b(os);
        if(!model.isRecordingInUse()) {
            os << "const unsigned int recordingTimestep = 0;" << std::endl;
        }
        os << "const unsigned long long b200Step = (unsigned long long)llround((double)t / " << Type::writeNumeric(model.getDT(), Type::Double) << ");" << std::endl;
        const std::string args = "t, recordingTimestep, b200Step, b200Seed";
        for(const auto &k : prevLaunches) {
            genLaunch(os, k, block, batchSize, args);
        }
        for(const auto &k : queueLaunches) {
            genLaunch(os, k, 32, 1, "");
        }
        genKernelTimerStart(os, "neuronUpdate", model.isTimingEnabled());
        for(const auto &k : neuronLaunches) {
            genLaunch(os, k, block, batchSize, args);
        }
        genKernelTimerStop(os, "neuronUpdate", model.isTimingEnabled(), true);
    }
}

//--------------------------------------------------------------------------
// Synapse update
//--------------------------------------------------------------------------
namespace
{
constexpr unsigned int SPIKE_LANES = 8;     // gridDim.z: a group's spike list is dealt to this many blocks per column block

//! Environment entries a presynaptic / synapse-dynamics body needs to deposit its output: fire-and-forget
//! fp32 additions (they compile to reductions; nothing reads the old value)
template<typename E, typename G>
void addOutputFunctions(E &env, G &sg, unsigned int batchSize)
{
    env.add(Type::getAddToPrePostDelay(sg.getScalarType()), "addToPostDelay",
            "atomicAdd(&$(_den_delay)[" + sg.getPostDenDelayIndex(batchSize, "$(id_post)", "$(1)") + "], $(0))");
    env.add(Type::getAddToPrePost(sg.getScalarType()), "addToPost",
            "atomicAdd(&$(_out_post)[" + sg.getPostISynIndex(batchSize, "$(id_post)") + "], $(0))");
    env.add(Type::getAddToPrePost(sg.getScalarType()), "addToPre",
            "atomicAdd(&$(_out_pre)[" + sg.getPreISynIndex(batchSize, "$(id_pre)") + "], $(0))");
}
}   // anonymous namespace

void Backend::genSynapseUpdate(CodeStream &os, FileStreamCreator, ModelSpecMerged &modelMerged,
                               BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const
{
    const ModelSpecInternal &model = modelMerged.getModel();
    const unsigned int batchSize = model.getBatchSize();
    const size_t block = blockSize();
    const std::string timeType = model.getTimePrecision().getName();
    const std::string dtLiteral = Type::writeNumeric(model.getDT(), model.getTimePrecision());
    const std::string kernelArgs = timeType + " t, unsigned long long b200Step, unsigned long long b200Seed";

    std::ostringstream kernelStream;
    CodeStream kernels(kernelStream);
    std::vector<KernelLaunch> delayLaunches, dynamicsLaunches, preLaunches, postLaunches;

    EnvironmentLibrary backendEnv(kernels, backendFunctions);
    EnvironmentLibrary mathsEnv(backendEnv, StandardLibrary::getMathsFunctions());
    EnvironmentLibrary kernelLibEnv(mathsEnv, randomFunctions(model.getPrecision()));

    auto beginKernel = [&](EnvironmentExternal &env, const std::string &structName, const std::string &arrayName,
                           const std::string &startName, size_t numGroups)
    {
        env.getStream() << "const unsigned int batch = blockIdx.y;" << std::endl;
        env.add(model.getTimePrecision().addConst(), "t", "t");
        env.add(Type::Uint32.addConst(), "batch", "batch");
        env.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
        genFindGroup(env.getStream(), structName, arrayName, startName, numGroups);
        env.add(Type::Uint32.addConst(), "id", "b200Local");
    };
    auto rngInitialiser = [](unsigned int stream, size_t index)
    {
        return "b200gen::Rng b200Rng = b200gen::simRng(b200Seed, " + std::to_string(stream + index) + "u + (b200Group << 20), b200Thread, $(batch), b200Step);";
    };

    // ---- dendritic delay pointers: one thread per group -------------------------------------------------------
    modelMerged.genMergedSynapseDendriticDelayUpdateGroups(
        *this, memorySpaces,
        [&](auto &sg)
        {
            const std::string idx = std::to_string(sg.getIndex());
            KernelLaunch launch;
            launch.name = "synapseDendriticDelayUpdateKernel" + idx;
            launch.numThreads = padTo(sg.getGroups().size(), 32);
            kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "()";
            {
                CodeStream::Scope b(kernelLibEnv.getStream());
                kernelLibEnv.getStream() << "const unsigned int b200Thread = (blockIdx.x * blockDim.x) + threadIdx.x;" << std::endl;
                kernelLibEnv.getStream() << "if(b200Thread < " << sg.getGroups().size() << ")";
                {
                    CodeStream::Scope b(kernelLibEnv.getStream());
                    EnvironmentExternal kernelEnv(kernelLibEnv);
                    kernelEnv.getStream() << "const MergedSynapseDendriticDelayUpdateGroup" << idx << " *group = &d_mergedSynapseDendriticDelayUpdateGroup" << idx << "[b200Thread];" << std::endl;
                    EnvironmentGroupMergedField<SynapseDendriticDelayUpdateGroupMerged> groupEnv(kernelEnv, sg);
                    buildStandardEnvironment(groupEnv, batchSize);
                    sg.generateSynapseUpdate(groupEnv);
                }
            }
            delayLaunches.push_back(launch);
        });

    // ---- synapse dynamics: one thread per synapse slot --------------------------------------------------------
    modelMerged.genMergedSynapseDynamicsGroups(
        *this, memorySpaces,
        [&](auto &sg)
        {
            const std::string idx = std::to_string(sg.getIndex());
            KernelLaunch launch;
            launch.name = "updateSynapseDynamicsKernel" + idx;
            launch.batched = true;
            launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedSynapseDynamicsGroupStartID" + idx, sg, block,
                                            [this](const SynapseGroupInternal &g)
                                            {
                                                return (size_t)g.getSrcNeuronGroup()->getNumNeurons() * getSynapticMatrixRowStride(g);
                                            });
            kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
            {
                CodeStream::Scope b(kernelLibEnv.getStream());
                EnvironmentExternal kernelEnv(kernelLibEnv);
                beginKernel(kernelEnv, "MergedSynapseDynamicsGroup" + idx, "d_mergedSynapseDynamicsGroup" + idx,
                            "d_mergedSynapseDynamicsGroupStartID" + idx, sg.getGroups().size());
                EnvironmentGroupMergedField<SynapseDynamicsGroupMerged> groupEnv(kernelEnv, sg);
                buildStandardEnvironment(groupEnv, batchSize);
                const bool sparse = (sg.getArchetype().getMatrixType() & SynapseMatrixConnectivity::SPARSE);
                if(!sparse && !(sg.getArchetype().getMatrixType() & SynapseMatrixConnectivity::DENSE)) {
                    throw std::runtime_error("B200 backend: synapse dynamics need SPARSE or DENSE connectivity");
                }
                groupEnv.print("if($(id) < ($(num_pre) * $(_row_stride)))");
                {
                    CodeStream::Scope b(groupEnv.getStream());
                    EnvironmentGroupMergedField<SynapseDynamicsGroupMerged> synEnv(groupEnv, sg);
                    synEnv.add(Type::Void, "_rng", "b200Rng", {synEnv.addInitialiser(rngInitialiser(STREAM_DYNAMICS, sg.getIndex()))});
                    synEnv.printLine("const unsigned int b200Row = $(id) / $(_row_stride);");
                    synEnv.printLine("const unsigned int b200Col = $(id) - (b200Row * $(_row_stride));");
                    synEnv.add(Type::Uint32.addConst(), "id_pre", "b200Row");
                    synEnv.add(Type::Uint32.addConst(), "id_syn", "$(id)");
                    if(sparse) {
                        synEnv.add(Type::Uint32.addConst(), "id_post", "$(_ind)[$(id)]");
                        synEnv.print("if(b200Col < $(_row_length)[b200Row])");
                    }
                    else {
                        synEnv.add(Type::Uint32.addConst(), "id_post", "b200Col");
                    }
                    {
                        CodeStream::Scope b(synEnv.getStream());
                        EnvironmentGroupMergedField<SynapseDynamicsGroupMerged> bodyEnv(synEnv, sg);
                        addOutputFunctions(bodyEnv, sg, batchSize);
                        sg.generateSynapseUpdate(*this, bodyEnv, batchSize, model.getDT());
                    }
                }
            }
            dynamicsLaunches.push_back(launch);
        });

    // ---- presynaptic update --------------------------------------------------------------------------------------------
    // A block column covers `block` synapses of a row (SPARSE: positions in the ragged row; DENSE / BITMASK:
    // target neurons); blockIdx.z = lane l takes spikes l, l + SPIKE_LANES, ...: the parallel width is
    // SPIKE_LANES x row stride, and each thread reads its synapse of every row it visits coalesced.
    modelMerged.genMergedPresynapticUpdateGroups(
        *this, memorySpaces,
        [&](auto &sg)
        {
            const std::string idx = std::to_string(sg.getIndex());
            const auto matrixType = sg.getArchetype().getMatrixType();
            const bool procedural = (matrixType & SynapseMatrixConnectivity::PROCEDURAL);
            const bool toeplitz = (matrixType & SynapseMatrixConnectivity::TOEPLITZ);
            const bool sparse = (matrixType & SynapseMatrixConnectivity::SPARSE);
            const bool bitmask = (matrixType & SynapseMatrixConnectivity::BITMASK);
            KernelLaunch launch;
            launch.name = "updatePresynapticKernel" + idx;
            launch.batched = true;
            // (PROCEDURAL: one block per group and spike lane; its threads walk the (spike, sub-row) items)
            launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedPresynapticUpdateGroupStartID" + idx, sg, block,
                                            [this, procedural, block](const SynapseGroupInternal &g)
                                            { return procedural ? block : getSynapticMatrixRowStride(g); });
            kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
            {
                CodeStream::Scope b(kernelLibEnv.getStream());
                EnvironmentExternal kernelEnv(kernelLibEnv);
                beginKernel(kernelEnv, "MergedPresynapticUpdateGroup" + idx, "d_mergedPresynapticUpdateGroup" + idx,
                            "d_mergedPresynapticUpdateGroupStartID" + idx, sg.getGroups().size());
                EnvironmentGroupMergedField<PresynapticUpdateGroupMerged> groupEnv(kernelEnv, sg);
                buildStandardEnvironment(groupEnv, batchSize);
                groupEnv.add(Type::Void, "_rng", "b200Rng", {groupEnv.addInitialiser(rngInitialiser(STREAM_PRESYNAPTIC, sg.getIndex()))});

                auto genEvents = [&](bool trueSpike)
                {
                    const std::string eventSuffix = trueSpike ? "" : "_event";
                    const bool delay = trueSpike ? sg.getArchetype().getSrcNeuronGroup()->isSpikeQueueRequired()
                                                 : sg.getArchetype().getSrcNeuronGroup()->isSpikeEventQueueRequired();
                    CodeStream::Scope b(groupEnv.getStream());
                    groupEnv.printLine("const unsigned int b200NumSpikes = $(_src_spk_cnt" + eventSuffix + ")[" + sg.getPreSlot(delay, batchSize) + "];");
                    groupEnv.print("if($(id) < $(_row_stride))");
                    {
                        CodeStream::Scope b(groupEnv.getStream());
                        groupEnv.getStream() << "for(unsigned int b200Spike = blockIdx.z; b200Spike < b200NumSpikes; b200Spike += gridDim.z)";
                        {
                            CodeStream::Scope b(groupEnv.getStream());
                            EnvironmentGroupMergedField<PresynapticUpdateGroupMerged> synEnv(groupEnv, sg);
                            // (initialisers are emitted before the body of an environment, in the order they were added)
                            synEnv.add(Type::Uint32.addConst(), "id_pre", "b200Pre",
                                       {synEnv.addInitialiser("const unsigned int b200Pre = $(_src_spk" + eventSuffix + ")["
                                                              + sg.getPreVarIndex(delay, batchSize, VarAccessDim::BATCH | VarAccessDim::ELEMENT, "b200Spike") + "];")});
                            const auto indexType = getSynapseIndexType(sg);
                            const std::string indexTypeName = indexType.getName();
                            synEnv.add(indexType.addConst(), "id_syn", "b200Syn",
                                       {synEnv.addInitialiser("const " + indexTypeName + " b200Syn = ((" + indexTypeName + ")$(id_pre) * $(_row_stride)) + $(id);")});
                            if(sparse) {
                                synEnv.print("if($(id) < $(_row_length)[$(id_pre)])");
                                synEnv.add(Type::Uint32.addConst(), "id_post", "b200Post",
                                           {synEnv.addInitialiser("const unsigned int b200Post = $(_ind)[$(id_syn)];")});
                            }
                            else if(bitmask) {
                                synEnv.printLine("const " + indexTypeName + " b200Gid = ((" + indexTypeName + ")$(id_pre) * $(_row_stride)) + $(id);");
                                synEnv.print("if(($(id) < $(num_post)) && ($(_gp)[b200Gid / 32] & (0x80000000 >> (b200Gid & 31))))");
                                synEnv.add(Type::Uint32.addConst(), "id_post", "$(id)");
                            }
                            else {
                                synEnv.print("if($(id) < $(num_post))");
                                synEnv.add(Type::Uint32.addConst(), "id_post", "$(id)");
                            }
                            {
                                CodeStream::Scope b(synEnv.getStream());
                                EnvironmentGroupMergedField<PresynapticUpdateGroupMerged> bodyEnv(synEnv, sg);
                                addOutputFunctions(bodyEnv, sg, batchSize);
                                if(trueSpike) {
                                    sg.generateSpikeUpdate(*this, bodyEnv, batchSize, model.getDT());
                                }
                                else {
                                    sg.generateSpikeEventUpdate(*this, bodyEnv, batchSize, model.getDT());
                                }
                            }
                        }
                    }
                };
                // The body that handles ONE synapse, as a string in which $(0) is the target and $(1).. the kernel
                // indices: connectivity that is regenerated on the fly (PROCEDURAL, TOEPLITZ) calls it as addSynapse(...)
                const auto addSynapseType = Type::ResolvedType::createFunction(
                    Type::Void, std::vector<Type::ResolvedType>{1ull + sg.getArchetype().getKernelSize().size(), Type::Uint32});
                auto genSynapseBody = [&](EnvironmentExternalBase &parent, bool trueSpike)
                {
                    std::ostringstream bodyStream;
                    CodeStream body(bodyStream);
                    {
                        CodeStream::Scope b(body);
                        EnvironmentExternal bodyEnv(parent, body);
                        bodyEnv.add(Type::Uint32.addConst(), "id_post", "b200Post",
                                    {bodyEnv.addInitialiser("const unsigned int b200Post = $(0);")});
                        for(size_t i = 0; i < sg.getArchetype().getKernelSize().size(); i++) {
                            const std::string iStr = std::to_string(i);
                            bodyEnv.add(Type::Uint32.addConst(), "id_kernel_" + iStr, "b200Kernel" + iStr,
                                        {bodyEnv.addInitialiser("const unsigned int b200Kernel" + iStr + " = $(" + std::to_string(i + 1) + ");")});
                        }
                        addOutputFunctions(bodyEnv, sg, batchSize);
                        if(trueSpike) {
                            sg.generateSpikeUpdate(*this, bodyEnv, batchSize, model.getDT());
                        }
                        else {
                            sg.generateSpikeEventUpdate(*this, bodyEnv, batchSize, model.getDT());
                        }
                    }
                    return bodyStream.str();
                };

                // PROCEDURAL (presynapticUpdateStrategySIMT.cc:425-561): an item is (spike, sub-row t of T); the row
                // of a spiking neuron is rebuilt by the snippet's row build code from a stream keyed on
                // (row, sub-row) alone, so it is the same row at every spike
                auto genProceduralEvents = [&](bool trueSpike)
                {
                    const std::string eventSuffix = trueSpike ? "" : "_event";
                    const bool delay = trueSpike ? sg.getArchetype().getSrcNeuronGroup()->isSpikeQueueRequired()
                                                 : sg.getArchetype().getSrcNeuronGroup()->isSpikeEventQueueRequired();
                    const size_t T = sg.getArchetype().getNumThreadsPerSpike();
                    const std::string Tstr = std::to_string(T) + "u";
                    CodeStream::Scope b(groupEnv.getStream());
                    groupEnv.printLine("const unsigned int b200NumSpikes = $(_src_spk_cnt" + eventSuffix + ")[" + sg.getPreSlot(delay, batchSize) + "];");
                    groupEnv.printLine("for(unsigned int b200Item = (blockIdx.z * blockDim.x) + $(id); b200Item < (b200NumSpikes * " + Tstr
                                       + "); b200Item += (gridDim.z * blockDim.x))");
                    {
                        CodeStream::Scope b(groupEnv.getStream());
                        EnvironmentGroupMergedField<PresynapticUpdateGroupMerged> synEnv(groupEnv, sg);
                        synEnv.add(Type::Uint32.addConst(), "_spike", "b200Spike",
                                   {synEnv.addInitialiser("const unsigned int b200Spike = b200Item / " + Tstr + ";")});
                        synEnv.add(Type::Uint32.addConst(), "_thread", "b200Sub",
                                   {synEnv.addInitialiser("const unsigned int b200Sub = b200Item % " + Tstr + ";")});
                        synEnv.add(Type::Uint32.addConst(), "id_pre", "b200Pre",
                                   {synEnv.addInitialiser("const unsigned int b200Pre = $(_src_spk" + eventSuffix + ")["
                                                          + sg.getPreVarIndex(delay, batchSize, VarAccessDim::BATCH | VarAccessDim::ELEMENT, "$(_spike)") + "];")});
                        synEnv.add(Type::Uint32.addConst(), "_num_post", "$(num_post)");
                        synEnv.add(Type::Void, "_rng", "b200RowRng",
                                   {synEnv.addInitialiser("b200gen::Rng b200RowRng = b200gen::initRng(b200Seed, " + std::to_string(STREAM_PROCEDURAL + sg.getIndex())
                                                          + "u + (b200Group << 20), ($(id_pre) * " + Tstr + ") + $(_thread));")});
                        const std::string body = genSynapseBody(synEnv, trueSpike);
                        {
                            EnvironmentExternal connEnv(synEnv);
                            connEnv.add(Type::Uint32.addConst(), "num_threads", std::to_string(T));
                            if(T > 1) {
                                const size_t perInit = connEnv.addInitialiser("const unsigned int b200PostPerSub = ($(_num_post) + " + Tstr + " - 1u) / " + Tstr + ";");
                                connEnv.add(Type::Uint32.addConst(), "id_post_begin", "b200PostBegin",
                                            {perInit, connEnv.addInitialiser("const unsigned int b200PostBegin = $(_thread) * b200PostPerSub;")});
                                connEnv.add(Type::Uint32.addConst(), "id_thread", "$(_thread)");
                                connEnv.add(Type::Uint32.addConst(), "num_post", "b200SubPost",
                                            {perInit, connEnv.addInitialiser("const unsigned int b200SubPost = (($(_thread) * b200PostPerSub) >= $(_num_post)) ? 0u : "
                                                                             "min(b200PostPerSub, $(_num_post) - ($(_thread) * b200PostPerSub));")});
                            }
                            else {
                                connEnv.add(Type::Uint32.addConst(), "id_post_begin", "0");
                                connEnv.add(Type::Uint32.addConst(), "id_thread", "0");
                            }
                            connEnv.add(addSynapseType, "addSynapse", body);
                            sg.generateProceduralConnectivity(connEnv);
                        }
                    }
                };

                // TOEPLITZ (presynapticUpdateStrategySIMT.cc:784-919): thread = diagonal of the kernel; the diagonal
                // build code loops over the spikes through for_each_synapse and calls addSynapse for each target
                auto genToeplitzEvents = [&](bool trueSpike)
                {
                    const std::string eventSuffix = trueSpike ? "" : "_event";
                    const bool delay = trueSpike ? sg.getArchetype().getSrcNeuronGroup()->isSpikeQueueRequired()
                                                 : sg.getArchetype().getSrcNeuronGroup()->isSpikeEventQueueRequired();
                    CodeStream::Scope b(groupEnv.getStream());
                    EnvironmentExternal toeplitzEnv(groupEnv);
                    toeplitzEnv.add(Type::Uint32.addConst(), "id_diag", "$(id)");
                    toeplitzEnv.add(Type::Uint32.addConst(), "id_pre", "b200Pre");
                    const std::string body = genSynapseBody(toeplitzEnv, trueSpike);
                    sg.generateToeplitzConnectivity(
                        toeplitzEnv,
                        [addSynapseType](auto &env, auto &errorHandler)
                        {
                            env.define(Transpiler::Token{Transpiler::Token::Type::IDENTIFIER, "addSynapse", 0}, addSynapseType, errorHandler);
                            env.define(Transpiler::Token{Transpiler::Token::Type::IDENTIFIER, "id_pre", 0}, Type::Uint32.addConst(), errorHandler);
                        },
                        [&](auto &env, auto generateBody)
                        {
                            env.printLine("const unsigned int b200NumSpikes = $(_src_spk_cnt" + eventSuffix + ")[" + sg.getPreSlot(delay, batchSize) + "];");
                            env.getStream() << "for(unsigned int b200Spike = blockIdx.z; b200Spike < b200NumSpikes; b200Spike += gridDim.z)";
                            {
                                CodeStream::Scope b(env.getStream());
                                EnvironmentGroupMergedField<PresynapticUpdateGroupMerged> spikeEnv(env, sg);
                                spikeEnv.printLine("const unsigned int b200Pre = $(_src_spk" + eventSuffix + ")["
                                                   + sg.getPreVarIndex(delay, batchSize, VarAccessDim::BATCH | VarAccessDim::ELEMENT, "b200Spike") + "];");
                                spikeEnv.add(Type::Uint32.addConst(), "id_pre", "b200Pre");
                                spikeEnv.print("if($(id) < $(_row_stride))");
                                {
                                    CodeStream::Scope b(spikeEnv.getStream());
                                    EnvironmentExternal bodyEnv(spikeEnv);
                                    bodyEnv.add(addSynapseType, "addSynapse", body);
                                    generateBody(bodyEnv);
                                }
                            }
                        });
                };

                if(sg.getArchetype().isPreSpikeEventRequired()) {
                    procedural ? genProceduralEvents(false) : toeplitz ? genToeplitzEvents(false) : genEvents(false);
                }
                if(sg.getArchetype().isPreSpikeRequired()) {
                    procedural ? genProceduralEvents(true) : toeplitz ? genToeplitzEvents(true) : genEvents(true);
                }
            }
            preLaunches.push_back(launch);
        });

    // ---- postsynaptic update: thread = position in the spiking target's column ---------------------------------
    modelMerged.genMergedPostsynapticUpdateGroups(
        *this, memorySpaces,
        [&](auto &sg)
        {
            const std::string idx = std::to_string(sg.getIndex());
            const bool sparse = (sg.getArchetype().getMatrixType() & SynapseMatrixConnectivity::SPARSE);
            KernelLaunch launch;
            launch.name = "updatePostsynapticKernel" + idx;
            launch.batched = true;
            launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedPostsynapticUpdateGroupStartID" + idx, sg, block,
                                            [](const SynapseGroupInternal &g)
                                            {
                                                return (g.getMatrixType() & SynapseMatrixConnectivity::SPARSE)
                                                    ? (size_t)g.getMaxSourceConnections() : (size_t)g.getSrcNeuronGroup()->getNumNeurons();
                                            });
            kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
            {
                CodeStream::Scope b(kernelLibEnv.getStream());
                EnvironmentExternal kernelEnv(kernelLibEnv);
                beginKernel(kernelEnv, "MergedPostsynapticUpdateGroup" + idx, "d_mergedPostsynapticUpdateGroup" + idx,
                            "d_mergedPostsynapticUpdateGroupStartID" + idx, sg.getGroups().size());
                EnvironmentGroupMergedField<PostsynapticUpdateGroupMerged> groupEnv(kernelEnv, sg);
                buildStandardEnvironment(groupEnv, batchSize);
                groupEnv.add(Type::Void, "_rng", "b200Rng", {groupEnv.addInitialiser(rngInitialiser(STREAM_POSTSYNAPTIC, sg.getIndex()))});

                auto genEvents = [&](bool trueSpike)
                {
                    const std::string eventSuffix = trueSpike ? "" : "_event";
                    const bool delay = trueSpike ? sg.getArchetype().getTrgNeuronGroup()->isSpikeQueueRequired()
                                                 : sg.getArchetype().getTrgNeuronGroup()->isSpikeEventQueueRequired();
                    CodeStream::Scope b(groupEnv.getStream());
                    groupEnv.printLine("const unsigned int b200NumSpikes = $(_trg_spk_cnt" + eventSuffix + ")[" + sg.getPostSlot(delay, batchSize) + "];");
                    groupEnv.print(sparse ? "if($(id) < $(_col_stride))" : "if($(id) < $(num_pre))");
                    {
                        CodeStream::Scope b(groupEnv.getStream());
                        groupEnv.getStream() << "for(unsigned int b200Spike = blockIdx.z; b200Spike < b200NumSpikes; b200Spike += gridDim.z)";
                        {
                            CodeStream::Scope b(groupEnv.getStream());
                            EnvironmentGroupMergedField<PostsynapticUpdateGroupMerged> synEnv(groupEnv, sg);
                            synEnv.add(Type::Uint32.addConst(), "id_post", "b200Post",
                                       {synEnv.addInitialiser("const unsigned int b200Post = $(_trg_spk" + eventSuffix + ")["
                                                              + sg.getPostVarIndex(delay, batchSize, VarAccessDim::BATCH | VarAccessDim::ELEMENT, "b200Spike") + "];")});
                            if(sparse) {
                                synEnv.print("if($(id) < $(_col_length)[$(id_post)])");
                                synEnv.add(Type::Uint32.addConst(), "id_syn", "b200Syn",
                                           {synEnv.addInitialiser("const unsigned int b200Syn = $(_remap)[($(id_post) * $(_col_stride)) + $(id)];")});
                                synEnv.add(Type::Uint32.addConst(), "id_pre", "b200Pre",
                                           {synEnv.addInitialiser("const unsigned int b200Pre = $(id_syn) / $(_row_stride);")});
                            }
                            else {
                                synEnv.add(Type::Uint32.addConst(), "id_syn", "b200Syn",
                                           {synEnv.addInitialiser("const unsigned int b200Syn = ($(id) * $(num_post)) + $(id_post);")});
                                synEnv.add(Type::Uint32.addConst(), "id_pre", "$(id)");
                            }
                            {
                                CodeStream::Scope b(synEnv.getStream());
                                EnvironmentGroupMergedField<PostsynapticUpdateGroupMerged> bodyEnv(synEnv, sg);
                                bodyEnv.add(Type::getAddToPrePost(sg.getScalarType()), "addToPre",
                                            "atomicAdd(&$(_out_pre)[" + sg.getPreISynIndex(batchSize, "$(id_pre)") + "], $(0))");
                                if(trueSpike) {
                                    sg.generateSpikeUpdate(*this, bodyEnv, batchSize, model.getDT());
                                }
                                else {
                                    sg.generateSpikeEventUpdate(*this, bodyEnv, batchSize, model.getDT());
                                }
                            }
                        }
                    }
                };
                if(sg.getArchetype().isPostSpikeEventRequired()) {
                    genEvents(false);
                }
                if(sg.getArchetype().isPostSpikeRequired()) {
                    genEvents(true);
                }
            }
            postLaunches.push_back(launch);
        });

    // ---- file -----------------------------------------------------------------------------------------------------------
    modelMerged.genMergedSynapseDendriticDelayUpdateStructs(os, *this);
    modelMerged.genMergedPresynapticUpdateGroupStructs(os, *this);
    modelMerged.genMergedPostsynapticUpdateGroupStructs(os, *this);
    modelMerged.genMergedSynapseDynamicsGroupStructs(os, *this);
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedSynapseDendriticDelayUpdateGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedPresynapticUpdateGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedPostsynapticUpdateGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedSynapseDynamicsGroups());
    preambleHandler(os);
    os << kernelStream.str();

    auto genLaneLaunch = [&](const KernelLaunch &k)
    {
        if(k.numThreads == 0) {
            return;
        }
        CodeStream::Scope b(os);
        os << "const dim3 threads(" << block << ", 1, 1);" << std::endl;
        os << "const dim3 grid(" << (k.numThreads / block) << ", " << batchSize << ", " << SPIKE_LANES << ");" << std::endl;
        os << k.name << "<<<grid, threads>>>(t, b200Step, b200Seed);" << std::endl;
        os << "CHECK_RUNTIME_ERRORS(cudaPeekAtLastError());" << std::endl;
    };
    os << "void updateSynapses(" << timeType << " t)";
    {
        CodeStream::Scope b(os);
        os << "const unsigned long long b200Step = (unsigned long long)llround((double)t / " << Type::writeNumeric(model.getDT(), Type::Double) << ");" << std::endl;
        for(const auto &k : delayLaunches) {
            genLaunch(os, k, 32, 1, "");
        }
        if(!dynamicsLaunches.empty()) {
            genKernelTimerStart(os, "synapseDynamics", model.isTimingEnabled());
            for(const auto &k : dynamicsLaunches) {
                genLaunch(os, k, block, batchSize, "t, b200Step, b200Seed");
            }
            genKernelTimerStop(os, "synapseDynamics", model.isTimingEnabled(), true);
        }
        if(!preLaunches.empty()) {
            genKernelTimerStart(os, "presynapticUpdate", model.isTimingEnabled());
            for(const auto &k : preLaunches) {
                genLaneLaunch(k);
            }
            genKernelTimerStop(os, "presynapticUpdate", model.isTimingEnabled(), true);
        }
        if(!postLaunches.empty()) {
            genKernelTimerStart(os, "postsynapticUpdate", model.isTimingEnabled());
            for(const auto &k : postLaunches) {
                genLaneLaunch(k);
            }
            genKernelTimerStop(os, "postsynapticUpdate", model.isTimingEnabled(), true);
        }
    }
}

//--------------------------------------------------------------------------
// Initialisation
//--------------------------------------------------------------------------
// Loop shapes the group emitters ask for.  The parallel dimension is the thread: a neuron for
// neuron variables, a target neuron (dense) or a position in the ragged row (sparse) for
// per-synapse variables; the emitters loop over the other dimension themselves.
void Backend::genPopVariableInit(EnvironmentExternalBase &env, HandlerEnv handler) const
{
    env.getStream() << "if(" << env["id"] << " == 0)";
    {
        CodeStream::Scope b(env.getStream());
        handler(env);
    }
}

void Backend::genVariableInit(EnvironmentExternalBase &env, const std::string&, const std::string&, HandlerEnv handler) const
{
    handler(env);       // the thread is the element
}

void Backend::genSparseSynapseVariableRowInit(EnvironmentExternalBase &env, HandlerEnv handler) const
{
    EnvironmentExternal varEnv(env);
    varEnv.add(Type::Uint32.addConst(), "id_syn", "b200InitSyn",
               {varEnv.addInitialiser("const unsigned int b200InitSyn = ($(id_pre) * $(_row_stride)) + $(id);")});
    handler(varEnv);
}

void Backend::genDenseSynapseVariableRowInit(EnvironmentExternalBase &env, HandlerEnv handler) const
{
    genSparseSynapseVariableRowInit(env, handler);
}

void Backend::genKernelSynapseVariableInit(EnvironmentExternalBase &env, SynapseInitGroupMerged&, HandlerEnv handler) const
{
    EnvironmentExternal varEnv(env);
    varEnv.add(Type::Uint32.addConst(), "id_syn", "$(id)");
    handler(varEnv);
}

void Backend::genKernelCustomUpdateVariableInit(EnvironmentExternalBase &env, CustomWUUpdateInitGroupMerged&, HandlerEnv handler) const
{
    EnvironmentExternal varEnv(env);
    varEnv.add(Type::Uint32.addConst(), "id_syn", "$(id)");
    handler(varEnv);
}

namespace
{
//! Expression for the flattened size of dimension `d` of a kernel-weight group
template<typename G>
std::string kernelDimension(const G &g, size_t d)
{
    return getKernelSize(g, d);
}

//! Body shared by synapse groups and custom WU updates with DENSE or KERNEL weights: thread = target
//! neuron (or flattened kernel element), the emitter loops over the source neurons
template<typename G>
void genDenseVarInit(const BackendBase &backend, EnvironmentExternalBase &env, G &g, unsigned int batchSize,
                     bool kernel, size_t kernelDimensions, const std::string &rngInit)
{
    env.print(kernel ? "if($(id) < $(_kernel_size))" : "if($(id) < $(num_post))");
    CodeStream::Scope b(env.getStream());
    EnvironmentGroupMergedField<G> initEnv(env, g);
    initEnv.add(Type::Void, "_rng", "b200Rng", {initEnv.addInitialiser(rngInit)});
    if(kernel) {
        for(size_t i = 0; i < kernelDimensions; i++) {
            std::ostringstream init;
            init << "const unsigned int b200Kernel" << i << " = ($(id)";
            if(i < (kernelDimensions - 1)) {
                init << " / (";
                for(size_t j = (kernelDimensions - 1); j > i; j--) {
                    init << kernelDimension(g, j);
                    if(j != (i + 1)) {
                        init << " * ";
                    }
                }
                init << ")";
            }
            init << ")";
            if(i > 0) {
                init << " % " << kernelDimension(g, i);
            }
            init << ";";
            initEnv.add(Type::Uint32.addConst(), "id_kernel_" + std::to_string(i), "b200Kernel" + std::to_string(i),
                        {initEnv.addInitialiser(init.str())});
        }
    }
    else {
        initEnv.add(Type::Uint32.addConst(), "id_post", "$(id)");
    }
    g.generateInit(backend, initEnv, batchSize);
}

//! Body shared by the SPARSE per-synapse initialisers: thread = position in the ragged row, loop over
//! the rows; `handler` adds per-synapse work of the backend's own (the column-major remap)
template<typename G, typename H>
void genSparseVarInit(const BackendBase &backend, EnvironmentExternalBase &env, G &g, unsigned int batchSize,
                      bool varInitRequired, H handler)
{
    env.printLine("unsigned int idx = $(id);");
    env.print("for(unsigned int b200Row = 0; b200Row < $(num_pre); b200Row++)");
    {
        CodeStream::Scope b(env.getStream());
        env.print("if($(id) < $(_row_length)[b200Row])");
        {
            CodeStream::Scope b(env.getStream());
            if(varInitRequired) {
                EnvironmentExternal initEnv(env);
                initEnv.add(Type::Uint32.addConst(), "id_pre", "b200Row");
                initEnv.add(Type::Uint32.addConst(), "id_post", "$(_ind)[idx]");
                g.generateInit(backend, initEnv, batchSize);
            }
            handler(env);
        }
        env.printLine("idx += $(_row_stride);");
    }
}
}   // anonymous namespace

void Backend::genInit(CodeStream &os, FileStreamCreator, ModelSpecMerged &modelMerged,
                      BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const
{
    const ModelSpecInternal &model = modelMerged.getModel();
    const unsigned int batchSize = model.getBatchSize();
    const size_t block = blockSize();
    const std::string dtLiteral = Type::writeNumeric(model.getDT(), model.getTimePrecision());

    std::ostringstream kernelStream;
    CodeStream kernels(kernelStream);
    std::vector<KernelLaunch> initLaunches, sparseLaunches;

    EnvironmentLibrary backendEnv(kernels, backendFunctions);
    EnvironmentLibrary mathsEnv(backendEnv, StandardLibrary::getMathsFunctions());
    EnvironmentLibrary kernelLibEnv(mathsEnv, randomFunctions(model.getPrecision()));

    auto rngInit = [](unsigned int stream, size_t index)
    {
        return "b200gen::Rng b200Rng = b200gen::initRng(b200Seed, " + std::to_string(stream + index) + "u + (b200Group << 20), b200Thread);";
    };
    // one kernel of one merged group: prologue + body
    auto genKernel = [&](auto &g, const std::string &kernelName, const std::string &typeName, auto getNumThreads,
                         std::vector<KernelLaunch> &launches, auto body)
    {
        const std::string idx = std::to_string(g.getIndex());
        KernelLaunch launch;
        launch.name = kernelName + idx;
        launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_merged" + typeName + "GroupStartID" + idx, g, block, getNumThreads);
        kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(unsigned long long b200Seed)";
        {
            CodeStream::Scope b(kernelLibEnv.getStream());
            EnvironmentExternal kernelEnv(kernelLibEnv);
            kernelEnv.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
            genFindGroup(kernelEnv.getStream(), "Merged" + typeName + "Group" + idx, "d_merged" + typeName + "Group" + idx,
                         "d_merged" + typeName + "GroupStartID" + idx, g.getGroups().size());
            kernelEnv.add(Type::Uint32.addConst(), "id", "b200Local");
            body(kernelEnv);
        }
        launches.push_back(launch);
    };

    // ---- neuron variables ------------------------------------------------------------------------------------
    modelMerged.genMergedNeuronInitGroups(
        *this, memorySpaces,
        [&](auto &n)
        {
            genKernel(n, "initializeNeuronKernel", "NeuronInit", [](const NeuronGroupInternal &ng){ return (size_t)ng.getNumNeurons(); }, initLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<NeuronInitGroupMerged> groupEnv(kernelEnv, n);
                          buildStandardEnvironment(groupEnv, batchSize);
                          groupEnv.print("if($(id) < $(num_neurons))");
                          {
                              CodeStream::Scope b(groupEnv.getStream());
                              EnvironmentGroupMergedField<NeuronInitGroupMerged> initEnv(groupEnv, n);
                              initEnv.add(Type::Void, "_rng", "b200Rng", {initEnv.addInitialiser(rngInit(STREAM_INIT_NEURON, n.getIndex()))});
                              n.generateInit(*this, initEnv, batchSize);
                          }
                      });
        });

    // ---- DENSE / KERNEL weight update variables -----------------------------------------------------------------
    modelMerged.genMergedSynapseInitGroups(
        *this, memorySpaces,
        [&](auto &s)
        {
            const bool kernel = (s.getArchetype().getMatrixType() & SynapseMatrixWeight::KERNEL);
            genKernel(s, "initializeSynapseKernel", "SynapseInit",
                      [](const SynapseGroupInternal &sg)
                      {
                          return (sg.getMatrixType() & SynapseMatrixWeight::KERNEL) ? (size_t)sg.getKernelSizeFlattened()
                                                                                    : (size_t)sg.getTrgNeuronGroup()->getNumNeurons();
                      },
                      initLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<SynapseInitGroupMerged> groupEnv(kernelEnv, s);
                          buildStandardEnvironment(groupEnv, batchSize);
                          genDenseVarInit(*this, groupEnv, s, batchSize, kernel, s.getArchetype().getKernelSize().size(),
                                          rngInit(STREAM_INIT_SYNAPSE, s.getIndex()));
                      });
        });

    // ---- custom update variables ---------------------------------------------------------------------------------
    modelMerged.genMergedCustomUpdateInitGroups(
        *this, memorySpaces,
        [&](auto &c)
        {
            genKernel(c, "initializeCustomUpdateKernel", "CustomUpdateInit", [](const CustomUpdateInternal &cg){ return (size_t)cg.getNumNeurons(); }, initLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<CustomUpdateInitGroupMerged> groupEnv(kernelEnv, c);
                          buildStandardEnvironment(groupEnv, batchSize);
                          groupEnv.print("if($(id) < $(num_neurons))");
                          {
                              CodeStream::Scope b(groupEnv.getStream());
                              EnvironmentGroupMergedField<CustomUpdateInitGroupMerged> initEnv(groupEnv, c);
                              initEnv.add(Type::Void, "_rng", "b200Rng", {initEnv.addInitialiser(rngInit(STREAM_INIT_CUSTOM, c.getIndex()))});
                              c.generateInit(*this, initEnv, batchSize);
                          }
                      });
        });
    modelMerged.genMergedCustomWUUpdateInitGroups(
        *this, memorySpaces,
        [&](auto &c)
        {
            const SynapseGroupInternal *sgInternal = c.getArchetype().getSynapseGroup();
            const bool kernel = (sgInternal->getMatrixType() & SynapseMatrixWeight::KERNEL);
            genKernel(c, "initializeCustomWUUpdateKernel", "CustomWUUpdateInit",
                      [](const CustomUpdateWUInternal &cg)
                      {
                          const auto *sg = cg.getSynapseGroup();
                          return (sg->getMatrixType() & SynapseMatrixWeight::KERNEL) ? (size_t)sg->getKernelSizeFlattened()
                                                                                     : (size_t)sg->getTrgNeuronGroup()->getNumNeurons();
                      },
                      initLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<CustomWUUpdateInitGroupMerged> groupEnv(kernelEnv, c);
                          buildStandardEnvironment(groupEnv, batchSize);
                          genDenseVarInit(*this, groupEnv, c, batchSize, kernel, sgInternal->getKernelSize().size(),
                                          rngInit(STREAM_INIT_CUSTOM_WU, c.getIndex()));
                      });
        });
    // ---- variables of custom connectivity updates: per source neuron, per target neuron -----------------------------
    modelMerged.genMergedCustomConnectivityUpdatePreInitGroups(
        *this, memorySpaces,
        [&](auto &c)
        {
            genKernel(c, "initializeCustomConnectivityPreKernel", "CustomConnectivityUpdatePreInit",
                      [](const CustomConnectivityUpdateInternal &cg){ return (size_t)cg.getSynapseGroup()->getSrcNeuronGroup()->getNumNeurons(); }, initLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<CustomConnectivityUpdatePreInitGroupMerged> groupEnv(kernelEnv, c);
                          buildStandardEnvironment(groupEnv);
                          groupEnv.print("if($(id) < $(num_neurons))");
                          {
                              CodeStream::Scope b(groupEnv.getStream());
                              EnvironmentGroupMergedField<CustomConnectivityUpdatePreInitGroupMerged> initEnv(groupEnv, c);
                              initEnv.add(Type::Void, "_rng", "b200Rng", {initEnv.addInitialiser(rngInit(STREAM_INIT_CCU_PRE, c.getIndex()))});
                              c.generateInit(*this, initEnv, batchSize);
                          }
                      });
        });
    modelMerged.genMergedCustomConnectivityUpdatePostInitGroups(
        *this, memorySpaces,
        [&](auto &c)
        {
            genKernel(c, "initializeCustomConnectivityPostKernel", "CustomConnectivityUpdatePostInit",
                      [](const CustomConnectivityUpdateInternal &cg){ return (size_t)cg.getSynapseGroup()->getTrgNeuronGroup()->getNumNeurons(); }, initLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<CustomConnectivityUpdatePostInitGroupMerged> groupEnv(kernelEnv, c);
                          buildStandardEnvironment(groupEnv);
                          groupEnv.print("if($(id) < $(num_neurons))");
                          {
                              CodeStream::Scope b(groupEnv.getStream());
                              EnvironmentGroupMergedField<CustomConnectivityUpdatePostInitGroupMerged> initEnv(groupEnv, c);
                              initEnv.add(Type::Void, "_rng", "b200Rng", {initEnv.addInitialiser(rngInit(STREAM_INIT_CCU_POST, c.getIndex()))});
                              c.generateInit(*this, initEnv, batchSize);
                          }
                      });
        });

    // ---- sparse / bitmask connectivity built on the device ------------------------------------------------------------
    modelMerged.genMergedSynapseConnectivityInitGroups(
        *this, memorySpaces,
        [&](auto &s)
        {
            const auto &connectInit = s.getArchetype().getSparseConnectivityInitialiser();
            const bool rowBuild = !Utils::areTokensEmpty(connectInit.getRowBuildCodeTokens());
            const bool sparse = (s.getArchetype().getMatrixType() & SynapseMatrixConnectivity::SPARSE);
            if(!sparse && !(s.getArchetype().getMatrixType() & SynapseMatrixConnectivity::BITMASK)) {
                throw std::runtime_error("Only BITMASK and SPARSE format connectivity can be generated using a connectivity initialiser");
            }
            genKernel(s, "initializeConnectivityKernel", "SynapseConnectivityInit",
                      [](const SynapseGroupInternal &sg)
                      {
                          return Utils::areTokensEmpty(sg.getSparseConnectivityInitialiser().getRowBuildCodeTokens())
                              ? (size_t)sg.getTrgNeuronGroup()->getNumNeurons() : (size_t)sg.getSrcNeuronGroup()->getNumNeurons();
                      },
                      initLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<SynapseConnectivityInitGroupMerged> groupEnv(kernelEnv, s);
                          buildStandardEnvironment(groupEnv, batchSize);
                          if(rowBuild) {
                              groupEnv.print("if($(id) < $(num_pre))");
                              groupEnv.add(Type::Uint32.addConst(), "id_pre", "$(id)");
                              groupEnv.add(Type::Uint32.addConst(), "id_post_begin", "0");
                          }
                          else {
                              groupEnv.print("if($(id) < $(num_post))");
                              groupEnv.add(Type::Uint32.addConst(), "id_post", "$(id)");
                              groupEnv.add(Type::Uint32.addConst(), "id_pre_begin", "0");
                          }
                          groupEnv.add(Type::Uint32.addConst(), "id_thread", "0");
                          groupEnv.add(Type::Uint32.addConst(), "num_threads", "1");
                          CodeStream::Scope b(groupEnv.getStream());

                          // what addSynapse(j[, kernel indices]) expands to
                          std::ostringstream addSynapseStream;
                          CodeStream addSynapse(addSynapseStream);
                          {
                              CodeStream::Scope b(addSynapse);
                              EnvironmentExternal addSynapseEnv(groupEnv, addSynapse);
                              if(rowBuild) {
                                  addSynapseEnv.add(Type::Uint32.addConst(), "id_post", "b200NewPost",
                                                    {addSynapseEnv.addInitialiser("const unsigned int b200NewPost = $(0);")});
                              }
                              else {
                                  addSynapseEnv.add(Type::Uint32.addConst(), "id_pre", "b200NewPre",
                                                    {addSynapseEnv.addInitialiser("const unsigned int b200NewPre = $(0);")});
                              }
                              if(sparse) {
                                  if(rowBuild) {
                                      // the thread owns the row: plain increment
                                      addSynapseEnv.add(Type::Uint32.addConst(), "id_syn", "b200NewSyn",
                                                        {addSynapseEnv.addInitialiser("const unsigned int b200NewSyn = ($(id_pre) * $(_row_stride)) + $(_row_length)[$(id_pre)];")});
                                      addSynapseEnv.printLine("$(_row_length)[$(id_pre)]++;");
                                  }
                                  else {
                                      addSynapseEnv.add(Type::Uint32.addConst(), "id_syn", "b200NewSyn",
                                                        {addSynapseEnv.addInitialiser("const unsigned int b200RowPos = atomicAdd(&$(_row_length)[$(id_pre)], 1);"),
                                                         addSynapseEnv.addInitialiser("const unsigned int b200NewSyn = ($(id_pre) * $(_row_stride)) + b200RowPos;")});
                                  }
                                  addSynapseEnv.printLine("$(_ind)[$(id_syn)] = $(id_post);");
                                  if(!s.getArchetype().getKernelSize().empty()) {
                                      EnvironmentGroupMergedField<SynapseConnectivityInitGroupMerged> kernelInitEnv(addSynapseEnv, s);
                                      for(size_t i = 0; i < s.getArchetype().getKernelSize().size(); i++) {
                                          const std::string iStr = std::to_string(i);
                                          kernelInitEnv.add(Type::Uint32.addConst(), "id_kernel_" + iStr, "b200NewKernel" + iStr,
                                                            {kernelInitEnv.addInitialiser("const unsigned int b200NewKernel" + iStr + " = $(" + std::to_string(i + 1) + ");")});
                                      }
                                      s.generateKernelInit(kernelInitEnv, 1);
                                  }
                              }
                              else {
                                  // word-packed bits, MSB first (single_threaded_cpu/backend.cc:2003-2006)
                                  const std::string indexTypeName = getSynapseIndexType(s).getName();
                                  if(rowBuild) {
                                      addSynapseEnv.printLine("const " + indexTypeName + " b200Gid = ((" + indexTypeName + ")$(id) * $(_row_stride)) + ($(0));");
                                  }
                                  else {
                                      addSynapseEnv.printLine("const " + indexTypeName + " b200Gid = ((" + indexTypeName + ")($(0)) * $(_row_stride)) + $(id);");
                                  }
                                  addSynapseEnv.printLine("atomicOr(&$(_gp)[b200Gid / 32], 0x80000000 >> (b200Gid & 31));");
                              }
                          }
                          const auto addSynapseType = Type::ResolvedType::createFunction(
                              Type::Void, std::vector<Type::ResolvedType>{1ull + s.getArchetype().getKernelSize().size(), Type::Uint32});
                          groupEnv.add(addSynapseType, "addSynapse", addSynapseStream.str());
                          groupEnv.add(Type::Void, "_rng", "b200Rng", {groupEnv.addInitialiser(rngInit(STREAM_INIT_CONNECT, s.getIndex()))});
                          if(rowBuild) {
                              if(sparse) {
                                  groupEnv.printLine("$(_row_length)[$(id)] = 0;");
                              }
                              s.generateSparseRowInit(groupEnv);
                          }
                          else {
                              s.generateSparseColumnInit(groupEnv);      // row lengths were zeroed when the array was created
                          }
                      });
        });

    // ---- after the connectivity exists (initializeSparse): per-synapse variables of SPARSE groups, remap -------
    modelMerged.genMergedSynapseSparseInitGroups(
        *this, memorySpaces,
        [&](auto &s)
        {
            genKernel(s, "initializeSparseKernel", "SynapseSparseInit", [](const SynapseGroupInternal &sg){ return (size_t)sg.getMaxConnections(); }, sparseLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<SynapseSparseInitGroupMerged> groupEnv(kernelEnv, s);
                          buildStandardEnvironment(groupEnv, batchSize);
                          groupEnv.add(Type::Void, "_rng", "b200Rng", {groupEnv.addInitialiser(rngInit(STREAM_INIT_SPARSE, s.getIndex()))});
                          const bool remap = s.getArchetype().isPostSpikeRequired() || s.getArchetype().isPostSpikeEventRequired();
                          genSparseVarInit(*this, groupEnv, s, batchSize, s.getArchetype().isWUVarInitRequired(),
                                           [&](EnvironmentExternalBase &env)
                                           {
                                               if(remap) {
                                                   // column-major view of the ragged matrix for postsynaptic learning
                                                   CodeStream::Scope b(env.getStream());
                                                   env.printLine("const unsigned int b200PostIndex = $(_ind)[idx];");
                                                   env.printLine("const unsigned int b200ColPos = atomicAdd(&$(_col_length)[b200PostIndex], 1);");
                                                   env.printLine("$(_remap)[(b200PostIndex * $(_col_stride)) + b200ColPos] = idx;");
                                               }
                                           });
                      });
        });
    modelMerged.genMergedCustomWUUpdateSparseInitGroups(
        *this, memorySpaces,
        [&](auto &c)
        {
            genKernel(c, "initializeCustomWUUpdateSparseKernel", "CustomWUUpdateSparseInit",
                      [](const CustomUpdateWUInternal &cg){ return (size_t)cg.getSynapseGroup()->getMaxConnections(); }, sparseLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<CustomWUUpdateSparseInitGroupMerged> groupEnv(kernelEnv, c);
                          buildStandardEnvironment(groupEnv, batchSize);
                          groupEnv.add(Type::Void, "_rng", "b200Rng", {groupEnv.addInitialiser(rngInit(STREAM_INIT_CUSTOM_WU_SPARSE, c.getIndex()))});
                          genSparseVarInit(*this, groupEnv, c, batchSize, true, [](EnvironmentExternalBase&){});
                      });
        });

    modelMerged.genMergedCustomConnectivityUpdateSparseInitGroups(
        *this, memorySpaces,
        [&](auto &c)
        {
            genKernel(c, "initializeCustomConnectivitySparseKernel", "CustomConnectivityUpdateSparseInit",
                      [](const CustomConnectivityUpdateInternal &cg){ return (size_t)cg.getSynapseGroup()->getMaxConnections(); }, sparseLaunches,
                      [&](EnvironmentExternal &kernelEnv)
                      {
                          EnvironmentGroupMergedField<CustomConnectivityUpdateSparseInitGroupMerged> groupEnv(kernelEnv, c);
                          buildStandardEnvironment(groupEnv);
                          groupEnv.add(Type::Void, "_rng", "b200Rng", {groupEnv.addInitialiser(rngInit(STREAM_INIT_CCU_SPARSE, c.getIndex()))});
                          genSparseVarInit(*this, groupEnv, c, batchSize, true, [](EnvironmentExternalBase&){});
                      });
        });

    // ---- file -----------------------------------------------------------------------------------------------------------
    os << "#include <iostream>" << std::endl;
    os << "#include <random>" << std::endl;
    os << "#include <cstdint>" << std::endl;
    os << std::endl;
    modelMerged.genMergedNeuronInitGroupStructs(os, *this);
    modelMerged.genMergedSynapseInitGroupStructs(os, *this);
    modelMerged.genMergedSynapseConnectivityInitGroupStructs(os, *this);
    modelMerged.genMergedSynapseSparseInitGroupStructs(os, *this);
    modelMerged.genMergedCustomUpdateInitGroupStructs(os, *this);
    modelMerged.genMergedCustomWUUpdateInitGroupStructs(os, *this);
    modelMerged.genMergedCustomWUUpdateSparseInitGroupStructs(os, *this);
    modelMerged.genMergedCustomConnectivityUpdatePreInitStructs(os, *this);
    modelMerged.genMergedCustomConnectivityUpdatePostInitStructs(os, *this);
    modelMerged.genMergedCustomConnectivityUpdateSparseInitStructs(os, *this);
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomConnectivityUpdatePreInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomConnectivityUpdatePostInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomConnectivityUpdateSparseInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedNeuronInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedSynapseInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedSynapseConnectivityInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedSynapseSparseInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomUpdateInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomWUUpdateInitGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomWUUpdateSparseInitGroups());
    preambleHandler(os);
    os << kernelStream.str();

    os << "void initialize()";
    {
        CodeStream::Scope b(os);
        genKernelTimerStart(os, "init", model.isTimingEnabled());
        for(const auto &k : initLaunches) {
            genLaunch(os, k, block, 1, "b200Seed");
        }
        genKernelTimerStop(os, "init", model.isTimingEnabled(), true);
    }
    os << std::endl;
    os << "void initializeSparse()";
    {
        CodeStream::Scope b(os);
        if(!sparseLaunches.empty()) {
            const bool timer = model.isTimingEnabled() && !modelMerged.getMergedSynapseSparseInitGroups().empty();
            genKernelTimerStart(os, "initSparse", timer);
            for(const auto &k : sparseLaunches) {
                genLaunch(os, k, block, 1, "b200Seed");
            }
            genKernelTimerStop(os, "initSparse", timer, true);
        }
    }
}

//--------------------------------------------------------------------------
// Custom updates
//--------------------------------------------------------------------------
void Backend::genCustomUpdate(CodeStream &os, FileStreamCreator, ModelSpecMerged &modelMerged,
                              BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const
{
    const ModelSpecInternal &model = modelMerged.getModel();
    const unsigned int batchSize = model.getBatchSize();
    const size_t block = blockSize();
    const std::string timeType = model.getTimePrecision().getName();
    const std::string dtLiteral = Type::writeNumeric(model.getDT(), model.getTimePrecision());
    const std::string kernelArgs = timeType + " t, unsigned long long b200Step, unsigned long long b200Seed";

    std::ostringstream kernelStream;
    CodeStream kernels(kernelStream);
    EnvironmentLibrary backendEnv(kernels, backendFunctions);
    EnvironmentLibrary mathsEnv(backendEnv, StandardLibrary::getMathsFunctions());
    EnvironmentLibrary kernelLibEnv(mathsEnv, randomFunctions(model.getPrecision()));

    // names of all custom update groups
    std::set<std::string> updateGroups;
    for(const auto &c : model.getCustomUpdates()) {
        updateGroups.insert(c.second.getUpdateGroupName());
    }
    for(const auto &c : model.getCustomWUUpdates()) {
        updateGroups.insert(c.second.getUpdateGroupName());
    }
    for(const auto &c : model.getCustomConnectivityUpdates()) {
        updateGroups.insert(c.second.getUpdateGroupName());
    }

    std::map<std::string, std::vector<KernelLaunch>> launches, transposeLaunches, remapLaunches;
    std::map<std::string, std::string> hostUpdates;
    for(const auto &g : updateGroups) {
        // ---- neuron-shaped custom updates ---------------------------------------------------------------------------
        modelMerged.genMergedCustomUpdateGroups(
            *this, memorySpaces, g,
            [&](auto &cg)
            {
                const std::string idx = std::to_string(cg.getIndex());
                const bool batchReduce = cg.getArchetype().isBatchReduction();
                const bool neuronReduce = cg.getArchetype().isNeuronReduction();
                const bool perElement = (cg.getArchetype().getDims() & VarAccessDim::ELEMENT);
                const bool batched = (cg.getArchetype().getDims() & VarAccessDim::BATCH) && (batchSize > 1);
                KernelLaunch launch;
                launch.name = "customUpdate" + g + "Kernel" + idx;
                // grid.y spans the batch unless the batch is what is being reduced
                launch.batched = batched && !batchReduce;
                launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedCustomUpdateGroupStartID" + idx, cg, block,
                                                [&](const CustomUpdateInternal &cu)
                                                {
                                                    return (neuronReduce || !perElement) ? (size_t)32 : (size_t)cu.getNumNeurons();
                                                });
                kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
                {
                    CodeStream::Scope b(kernelLibEnv.getStream());
                    EnvironmentExternal kernelEnv(kernelLibEnv);
                    kernelEnv.add(model.getTimePrecision().addConst(), "t", "t");
                    kernelEnv.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
                    genFindGroup(kernelEnv.getStream(), "MergedCustomUpdateGroup" + idx, "d_mergedCustomUpdateGroup" + idx,
                                 "d_mergedCustomUpdateGroupStartID" + idx, cg.getGroups().size());
                    kernelEnv.add(Type::Uint32.addConst(), "id", "b200Local");
                    EnvironmentGroupMergedField<CustomUpdateGroupMerged> groupEnv(kernelEnv, cg);
                    buildSizeEnvironment(groupEnv);
                    if(batchReduce) {
                        // one thread per element walks the batch (values of one element are a stride apart,
                        // neighbouring threads read neighbouring addresses)
                        groupEnv.print("if($(id) < $(num_neurons))");
                        CodeStream::Scope b(groupEnv.getStream());
                        const auto reductionTargets = genInitReductionTargets(groupEnv.getStream(), cg, batchSize, groupEnv["id"]);
                        groupEnv.getStream() << "for(unsigned int batch = 0; batch < " << batchSize << "; batch++)";
                        {
                            CodeStream::Scope b(groupEnv.getStream());
                            EnvironmentGroupMergedField<CustomUpdateGroupMerged> batchEnv(groupEnv, cg);
                            batchEnv.add(Type::Uint32.addConst(), "batch", "batch");
                            buildStandardEnvironment(batchEnv, batchSize);
                            cg.generateCustomUpdate(batchEnv, batchSize,
                                                    [&reductionTargets, this](auto &env, const auto&)
                                                    {
                                                        for(const auto &r : reductionTargets) {
                                                            env.printLine(getReductionOperation("_lr" + r.name, "$(" + r.name + ")", r.access, r.type) + ";");
                                                        }
                                                    });
                        }
                        for(const auto &r : reductionTargets) {
                            groupEnv.printLine("group->" + r.name + "[" + r.index + "] = _lr" + r.name + ";");
                        }
                    }
                    else if(neuronReduce) {
                        // one warp per batch element strides over the neurons, then combines its lanes
                        groupEnv.getStream() << "const unsigned int batch = blockIdx.y;" << std::endl;
                        groupEnv.add(Type::Uint32.addConst(), "batch", batched ? "batch" : "0");
                        groupEnv.print("if($(id) < 32)");
                        CodeStream::Scope b(groupEnv.getStream());
                        groupEnv.printLine("const unsigned int b200Lane = $(id);");
                        EnvironmentGroupMergedField<CustomUpdateGroupMerged> batchEnv(groupEnv, cg);
                        buildStandardEnvironment(batchEnv, batchSize);
                        const auto reductionTargets = genInitReductionTargets(batchEnv.getStream(), cg, batchSize);
                        batchEnv.print("for(unsigned int b200Index = b200Lane; b200Index < $(num_neurons); b200Index += 32)");
                        {
                            CodeStream::Scope b(batchEnv.getStream());
                            batchEnv.add(Type::Uint32.addConst(), "id", "b200Index");
                            cg.generateCustomUpdate(batchEnv, batchSize,
                                                    [&reductionTargets, this](auto &env, const auto&)
                                                    {
                                                        for(const auto &r : reductionTargets) {
                                                            env.printLine(getReductionOperation("_lr" + r.name, "$(" + r.name + ")", r.access, r.type) + ";");
                                                        }
                                                    });
                        }
                        for(const auto &r : reductionTargets) {
                            for(int offset = 16; offset > 0; offset /= 2) {
                                batchEnv.getStream() << getReductionOperation("_lr" + r.name, "__shfl_down_sync(0xFFFFFFFF, _lr" + r.name + ", " + std::to_string(offset) + ")",
                                                                              r.access, r.type) << ";" << std::endl;
                            }
                        }
                        batchEnv.getStream() << "if(b200Lane == 0)";
                        {
                            CodeStream::Scope b(batchEnv.getStream());
                            for(const auto &r : reductionTargets) {
                                batchEnv.printLine("group->" + r.name + "[" + r.index + "] = _lr" + r.name + ";");
                            }
                        }
                    }
                    else {
                        groupEnv.getStream() << "const unsigned int batch = blockIdx.y;" << std::endl;
                        groupEnv.add(Type::Uint32.addConst(), "batch", batched ? "batch" : "0");
                        if(!perElement) {
                            // one value per population (and batch element): the first thread does it
                            groupEnv.print("if($(id) == 0)");
                        }
                        else {
                            groupEnv.print("if($(id) < $(num_neurons))");
                        }
                        CodeStream::Scope b(groupEnv.getStream());
                        EnvironmentGroupMergedField<CustomUpdateGroupMerged> batchEnv(groupEnv, cg);
                        buildStandardEnvironment(batchEnv, batchSize);
                        cg.generateCustomUpdate(batchEnv, batchSize, [](auto&, auto&){});
                    }
                }
                launches[g].push_back(launch);
            });

        // ---- per-synapse custom updates -------------------------------------------------------------------------------
        modelMerged.genMergedCustomUpdateWUGroups(
            *this, memorySpaces, g,
            [&](auto &cg)
            {
                const std::string idx = std::to_string(cg.getIndex());
                const SynapseGroupInternal *sg = cg.getArchetype().getSynapseGroup();
                const bool batchReduce = cg.getArchetype().isBatchReduction();
                const bool batched = (cg.getArchetype().getDims() & VarAccessDim::BATCH) && (batchSize > 1);
                KernelLaunch launch;
                launch.name = "customUpdateWU" + g + "Kernel" + idx;
                launch.batched = batched && !batchReduce;
                launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedCustomUpdateWUGroupStartID" + idx, cg, block,
                                                [this](const CustomUpdateWUInternal &cu)
                                                {
                                                    const auto *s = cu.getSynapseGroup();
                                                    return (s->getMatrixType() & SynapseMatrixWeight::KERNEL)
                                                        ? (size_t)s->getKernelSizeFlattened()
                                                        : (size_t)s->getSrcNeuronGroup()->getNumNeurons() * getSynapticMatrixRowStride(*s);
                                                });
                kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
                {
                    CodeStream::Scope b(kernelLibEnv.getStream());
                    EnvironmentExternal kernelEnv(kernelLibEnv);
                    kernelEnv.add(model.getTimePrecision().addConst(), "t", "t");
                    kernelEnv.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
                    genFindGroup(kernelEnv.getStream(), "MergedCustomUpdateWUGroup" + idx, "d_mergedCustomUpdateWUGroup" + idx,
                                 "d_mergedCustomUpdateWUGroupStartID" + idx, cg.getGroups().size());
                    kernelEnv.add(Type::Uint32.addConst(), "id", "b200Local");
                    EnvironmentGroupMergedField<CustomUpdateWUGroupMerged> groupEnv(kernelEnv, cg);
                    buildSizeEnvironment(groupEnv);
                    if(!batchReduce) {
                        groupEnv.getStream() << "const unsigned int batch = blockIdx.y;" << std::endl;
                        groupEnv.add(Type::Uint32.addConst(), "batch", batched ? "batch" : "0");
                    }
                    groupEnv.print("if($(id) < $(_size))");
                    {
                        CodeStream::Scope b(groupEnv.getStream());
                        EnvironmentGroupMergedField<CustomUpdateWUGroupMerged> synEnv(groupEnv, cg);
                        if(sg->getMatrixType() & SynapseMatrixWeight::KERNEL) {
                            synEnv.add(Type::Uint32.addConst(), "id_kernel", "$(id)");
                        }
                        else if(sg->getMatrixType() & SynapseMatrixConnectivity::SPARSE) {
                            synEnv.printLine("const unsigned int b200Row = $(id) / $(_row_stride);");
                            synEnv.printLine("const unsigned int b200Col = $(id) - (b200Row * $(_row_stride));");
                            synEnv.add(Type::Uint32.addConst(), "id_pre", "b200Row");
                            synEnv.add(Type::Uint32.addConst(), "id_post", "$(_ind)[$(id)]");
                            synEnv.print("if(b200Col < $(_row_length)[b200Row])");
                        }
                        else {
                            synEnv.add(Type::Uint32.addConst(), "id_pre", "b200Pre",
                                       {synEnv.addInitialiser("const unsigned int b200Pre = $(id) / $(_row_stride);")});
                            synEnv.add(Type::Uint32.addConst(), "id_post", "b200Post",
                                       {synEnv.addInitialiser("const unsigned int b200Post = $(id) % $(_row_stride);")});
                        }
                        CodeStream::Scope b2(synEnv.getStream());
                        synEnv.add(Type::Uint32.addConst(), "id_syn", "$(id)");
                        const auto reductionTargets = genInitReductionTargets(synEnv.getStream(), cg, batchSize, synEnv["id_syn"]);
                        if(batchReduce) {
                            synEnv.getStream() << "for(unsigned int batch = 0; batch < " << batchSize << "; batch++)";
                            synEnv.getStream() << CodeStream::OB(9100);
                            synEnv.add(Type::Uint32.addConst(), "batch", "batch");
                        }
                        {
                            EnvironmentGroupMergedField<CustomUpdateWUGroupMerged> batchEnv(synEnv, cg);
                            buildStandardEnvironment(batchEnv, batchSize);
                            cg.generateCustomUpdate(batchEnv, batchSize,
                                                    [&reductionTargets, this](auto &env, auto &c)
                                                    {
                                                        if(c.getArchetype().isBatchReduction()) {
                                                            for(const auto &r : reductionTargets) {
                                                                env.printLine(getReductionOperation("_lr" + r.name, "$(" + r.name + ")", r.access, r.type) + ";");
                                                            }
                                                        }
                                                    });
                        }
                        if(batchReduce) {
                            synEnv.getStream() << CodeStream::CB(9100);
                            for(const auto &r : reductionTargets) {
                                synEnv.printLine("group->" + r.name + "[" + r.index + "] = _lr" + r.name + ";");
                            }
                        }
                    }
                }
                launches[g].push_back(launch);
            });

        // ---- per-synapse custom updates that also write the transpose of one variable (DENSE only) -----------
        // thread = synapse of the forward matrix; the transposed element is written straight from the register
        // (rows of the transpose are a stride apart: the matrices these updates run on fit L2)
        modelMerged.genMergedCustomUpdateTransposeWUGroups(
            *this, memorySpaces, g,
            [&](auto &cg)
            {
                const std::string idx = std::to_string(cg.getIndex());
                const bool batched = (cg.getArchetype().getDims() & VarAccessDim::BATCH) && (batchSize > 1);
                KernelLaunch launch;
                launch.name = "customUpdateTransposeWU" + g + "Kernel" + idx;
                launch.batched = batched;
                launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedCustomUpdateTransposeWUGroupStartID" + idx, cg, block,
                                                [](const CustomUpdateWUInternal &cu)
                                                {
                                                    const auto *s = cu.getSynapseGroup();
                                                    return (size_t)s->getSrcNeuronGroup()->getNumNeurons() * s->getTrgNeuronGroup()->getNumNeurons();
                                                });
                kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
                {
                    CodeStream::Scope b(kernelLibEnv.getStream());
                    EnvironmentExternal kernelEnv(kernelLibEnv);
                    kernelEnv.add(model.getTimePrecision().addConst(), "t", "t");
                    kernelEnv.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
                    genFindGroup(kernelEnv.getStream(), "MergedCustomUpdateTransposeWUGroup" + idx, "d_mergedCustomUpdateTransposeWUGroup" + idx,
                                 "d_mergedCustomUpdateTransposeWUGroupStartID" + idx, cg.getGroups().size());
                    kernelEnv.add(Type::Uint32.addConst(), "id", "b200Local");
                    EnvironmentGroupMergedField<CustomUpdateTransposeWUGroupMerged> groupEnv(kernelEnv, cg);
                    buildSizeEnvironment(groupEnv);
                    groupEnv.getStream() << "const unsigned int batch = blockIdx.y;" << std::endl;
                    groupEnv.add(Type::Uint32.addConst(), "batch", batched ? "batch" : "0");
                    EnvironmentGroupMergedField<CustomUpdateTransposeWUGroupMerged> batchEnv(groupEnv, cg);
                    buildStandardEnvironment(batchEnv, batchSize);
                    const std::string transposeVarName = cg.addTransposeField(batchEnv);
                    batchEnv.print("if($(id) < ($(num_pre) * $(num_post)))");
                    {
                        CodeStream::Scope b(batchEnv.getStream());
                        EnvironmentGroupMergedField<CustomUpdateTransposeWUGroupMerged> synEnv(batchEnv, cg);
                        synEnv.add(Type::Uint32.addConst(), "id_pre", "b200Pre",
                                   {synEnv.addInitialiser("const unsigned int b200Pre = $(id) / $(num_post);")});
                        synEnv.add(Type::Uint32.addConst(), "id_post", "b200Post",
                                   {synEnv.addInitialiser("const unsigned int b200Post = $(id) % $(num_post);")});
                        synEnv.add(Type::Uint32.addConst(), "id_syn", "$(id)");
                        cg.generateCustomUpdate(synEnv, batchSize,
                                                [&transposeVarName, batched](auto &env, const auto&)
                                                {
                                                    env.print("$(" + transposeVarName + "_transpose)[");
                                                    if(batched) {
                                                        env.print("$(_batch_offset) + ");
                                                    }
                                                    env.printLine("($(id_post) * $(num_pre)) + $(id_pre)] = $(" + transposeVarName + ");");
                                                });
                    }
                }
                transposeLaunches[g].push_back(launch);
            });

        // ---- custom connectivity updates: thread = row; the row update code adds and removes synapses of its row ----
        modelMerged.genMergedCustomConnectivityUpdateGroups(
            *this, memorySpaces, g,
            [&](auto &cg)
            {
                const std::string idx = std::to_string(cg.getIndex());
                KernelLaunch launch;
                launch.name = "customConnectivityUpdate" + g + "Kernel" + idx;
                launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_mergedCustomConnectivityUpdateGroupStartID" + idx, cg, block,
                                                [](const CustomConnectivityUpdateInternal &cu)
                                                { return (size_t)cu.getSynapseGroup()->getSrcNeuronGroup()->getNumNeurons(); });
                kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
                {
                    CodeStream::Scope b(kernelLibEnv.getStream());
                    EnvironmentExternal kernelEnv(kernelLibEnv);
                    kernelEnv.add(model.getTimePrecision().addConst(), "t", "t");
                    kernelEnv.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
                    genFindGroup(kernelEnv.getStream(), "MergedCustomConnectivityUpdateGroup" + idx, "d_mergedCustomConnectivityUpdateGroup" + idx,
                                 "d_mergedCustomConnectivityUpdateGroupStartID" + idx, cg.getGroups().size());
                    kernelEnv.add(Type::Uint32.addConst(), "id", "b200Local");
                    EnvironmentGroupMergedField<CustomConnectivityUpdateGroupMerged> groupEnv(kernelEnv, cg);
                    buildStandardEnvironment(groupEnv);
                    groupEnv.print("if($(id) < $(num_pre))");
                    {
                        CodeStream::Scope b(groupEnv.getStream());
                        EnvironmentGroupMergedField<CustomConnectivityUpdateGroupMerged> validEnv(groupEnv, cg);
                        validEnv.add(Type::Uint32.addConst(), "id_pre", "$(id)");
                        // a stream per (row, update): stateless, where the reference keeps a generator state per row
                        validEnv.add(Type::Void, "_rng", "b200Rng",
                                     {validEnv.addInitialiser("b200gen::Rng b200Rng = b200gen::simRng(b200Seed, " + std::to_string(STREAM_CCU + cg.getIndex())
                                                              + "u + (b200Group << 20), b200Thread, 0u, b200Step);")});
                        cg.generateUpdate(*this, validEnv, batchSize);
                    }
                }
                launches[g].push_back(launch);
            });

        // ---- column-major view rebuilt after the rows changed: column lengths to zero, then one pass over the rows ----
        modelMerged.genMergedCustomConnectivityRemapUpdateGroups(
            *this, memorySpaces, g,
            [&](auto &cg)
            {
                const std::string idx = std::to_string(cg.getIndex());
                KernelLaunch zero, remap;
                zero.name = "customConnectivityRemapZero" + g + "Kernel" + idx;
                remap.name = "customConnectivityRemap" + g + "Kernel" + idx;
                for(int pass = 0; pass < 2; pass++) {
                    KernelLaunch &launch = pass ? remap : zero;
                    launch.numThreads = genStartIDs(kernelLibEnv.getStream(), "d_" + launch.name + "StartID", cg, block,
                                                    [pass](const CustomConnectivityUpdateInternal &cu)
                                                    {
                                                        return pass ? (size_t)cu.getSynapseGroup()->getMaxConnections()
                                                                    : (size_t)cu.getSynapseGroup()->getTrgNeuronGroup()->getNumNeurons();
                                                    });
                    kernelLibEnv.getStream() << "extern \"C\" __global__ void " << launch.name << "(" << kernelArgs << ")";
                    CodeStream::Scope b(kernelLibEnv.getStream());
                    EnvironmentExternal kernelEnv(kernelLibEnv);
                    genFindGroup(kernelEnv.getStream(), "MergedCustomConnectivityRemapUpdateGroup" + idx, "d_mergedCustomConnectivityRemapUpdateGroup" + idx,
                                 "d_" + launch.name + "StartID", cg.getGroups().size());
                    kernelEnv.add(Type::Uint32.addConst(), "id", "b200Local");
                    EnvironmentGroupMergedField<CustomConnectivityRemapUpdateGroupMerged> groupEnv(kernelEnv, cg);
                    buildStandardEnvironment(groupEnv);
                    if(pass == 0) {
                        groupEnv.print("if($(id) < $(num_post))");
                        CodeStream::Scope b(groupEnv.getStream());
                        groupEnv.printLine("$(_col_length)[$(id)] = 0;");
                    }
                    else {
                        groupEnv.printLine("unsigned int idx = $(id);");
                        groupEnv.print("for(unsigned int b200Row = 0; b200Row < $(num_pre); b200Row++)");
                        CodeStream::Scope b(groupEnv.getStream());
                        groupEnv.print("if($(id) < $(_row_length)[b200Row])");
                        {
                            CodeStream::Scope b(groupEnv.getStream());
                            groupEnv.printLine("const unsigned int b200PostIndex = $(_ind)[idx];");
                            groupEnv.printLine("const unsigned int b200ColPos = atomicAdd(&$(_col_length)[b200PostIndex], 1);");
                            groupEnv.printLine("$(_remap)[(b200PostIndex * $(_col_stride)) + b200ColPos] = idx;");
                        }
                        groupEnv.printLine("idx += $(_row_stride);");
                    }
                }
                remapLaunches[g].push_back(zero);
                remapLaunches[g].push_back(remap);
            });

        // ---- host update code of custom connectivity updates: runs on the host before the kernels ------------------
        {
            std::ostringstream hostStream;
            CodeStream host(hostStream);
            {
                // (an environment writes what it has gathered when it goes out of scope)
                EnvironmentExternal hostEnv(host);
                hostEnv.add(model.getTimePrecision().addConst(), "t", "t");
                hostEnv.add(model.getTimePrecision().addConst(), "dt", dtLiteral);
                modelMerged.genMergedCustomConnectivityHostUpdateGroups(
                    *this, memorySpaces, g,
                    [&](auto &c)
                    {
                        c.generateUpdate(*this, hostEnv);
                    });
            }
            hostUpdates[g] = hostStream.str();
        }
    }

    // ---- file -----------------------------------------------------------------------------------------------------------
    modelMerged.genMergedCustomUpdateStructs(os, *this);
    modelMerged.genMergedCustomUpdateWUStructs(os, *this);
    modelMerged.genMergedCustomUpdateTransposeWUStructs(os, *this);
    modelMerged.genMergedCustomConnectivityUpdateStructs(os, *this);
    modelMerged.genMergedCustomConnectivityRemapUpdateStructs(os, *this);
    modelMerged.genMergedCustomConnectivityHostUpdateStructs(os, *this);
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomUpdateGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomUpdateWUGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomUpdateTransposeWUGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomConnectivityUpdateGroups());
    genDeviceStructArrayPush(os, *this, modelMerged.getMergedCustomConnectivityRemapUpdateGroups());
    genHostStructArrayPush(os, *this, modelMerged.getMergedCustomConnectivityHostUpdateGroups());
    preambleHandler(os);
    os << kernelStream.str();
    for(const auto &g : updateGroups) {
        os << "void update" << g << "(unsigned long long timestep)";
        CodeStream::Scope b(os);
        os << "const " << timeType << " t = timestep * " << dtLiteral << ";" << std::endl;
        os << "const unsigned long long b200Step = timestep;" << std::endl;
        if(!hostUpdates[g].empty()) {
            os << hostUpdates[g];
        }
        genKernelTimerStart(os, "customUpdate" + g, model.isTimingEnabled());
        for(const auto &k : launches[g]) {
            genLaunch(os, k, block, batchSize, "t, b200Step, b200Seed");
        }
        genKernelTimerStop(os, "customUpdate" + g, model.isTimingEnabled(), true);
        if(!transposeLaunches[g].empty()) {
            genKernelTimerStart(os, "customUpdate" + g + "Transpose", model.isTimingEnabled());
            for(const auto &k : transposeLaunches[g]) {
                genLaunch(os, k, block, batchSize, "t, b200Step, b200Seed");
            }
            genKernelTimerStop(os, "customUpdate" + g + "Transpose", model.isTimingEnabled(), true);
        }
        if(!remapLaunches[g].empty()) {
            genKernelTimerStart(os, "customUpdate" + g + "Remap", model.isTimingEnabled());
            for(const auto &k : remapLaunches[g]) {
                genLaunch(os, k, block, 1, "t, b200Step, b200Seed");
            }
            genKernelTimerStop(os, "customUpdate" + g + "Remap", model.isTimingEnabled(), true);
        }
    }
}
}   // namespace GeNN::CodeGenerator::B200
