// B200 code-generation backend for GeNN: a plug-in behind GeNN::CodeGenerator::BackendBase
// (include/genn/genn/code_generator/backendBase.h:127-486) that emits sm_100a CUDA for the
// per-timestep path and drives it through the unmodified GeNN runtime.
//
// What it replaces: the reference's BackendSIMT / BackendCUDAHIP / CUDA::Backend stack
// (src/genn/genn/code_generator/backendSIMT.cc, backendCUDAHIP.cc, src/genn/backends/cuda).
// What it keeps: GeNN's model description, transpiler, group merging and runtime.  The model's
// code strings reach the kernels through GeNN's own emitters (generateNeuronUpdate,
// generateSpikeUpdate ...), which this backend calls with its own environments, so ANY model that
// GeNN can describe is inlined into the kernel scaffolds below, not only the built-in ones.
//
// Kernel scaffolds (all generated text; the device helpers they call live in
// include/genn_b200_gen.cuh):
//  * one kernel per merged group; a thread finds its group by binary search over start ids
//    that are literals in the generated code;
//  * neuron update: warp-level spike compaction (ballot + one atomic per spiking warp, ids in
//    ascending order inside a warp), recording words written straight from the ballot;
//  * presynaptic update, SPARSE: one warp per (spike, 32-synapse chunk of its row), so the
//    parallel width grows with the number of spikes instead of being capped at the longest row;
//    DENSE / BITMASK: one thread per target neuron looping over the spike list;
//  * random numbers: stateless Philox4x32-10 keyed on (seed, group, neuron, time step): no
//    per-neuron generator state is read or written.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>

#include "varAccess.h"
#include "code_generator/backendBase.h"
#include "code_generator/environment.h"
#include "runtime/runtime.h"

namespace filesystem
{
class path;
}

namespace GeNN::CodeGenerator::B200
{
struct Preferences : public PreferencesBase
{
    //! CUDA device the generated code selects in allocateMem
    int deviceID = 0;

    //! Threads per block of every generated kernel (a multiple of 32)
    unsigned int blockSize = 128;

    //! Directory holding genn_b200_gen.cuh; empty = the include directory beside this library
    std::string includePath;

    //! nvcc executable used by the generated Makefile
    std::string nvccPath = "/usr/local/cuda/bin/nvcc";

    void updateHash(boost::uuids::detail::sha1 &hash) const;
};

class State : public Runtime::StateBase
{
};

//! Device + page-locked host memory behind Runtime::ArrayBase (runtime.h:95-182)
class Array : public Runtime::ArrayBase
{
public:
    Array(const Type::ResolvedType &type, size_t count, VarLocation location, bool uninitialized);
    virtual ~Array();

    virtual void allocate(size_t count) final;
    virtual void free() final;
    virtual void pushToDevice() final;
    virtual void pullFromDevice() final;
    virtual void pushSlice1DToDevice(size_t offset, size_t count) final;
    virtual void pullSlice1DFromDevice(size_t offset, size_t count) final;
    virtual void memsetDeviceObject(int value) final;
    virtual void serialiseDeviceObject(std::vector<std::byte> &bytes, bool pointerToPointer) const final;
    virtual void serialiseHostObject(std::vector<std::byte> &bytes, bool pointerToPointer) const final;

    std::byte *getDevicePointer() const { return m_DevicePointer; }

private:
    std::byte *m_DevicePointer = nullptr;
};

class Backend : public BackendBase
{
public:
    Backend(const Preferences &preferences);

    // ---- code emission ---------------------------------------------------------------------------
    virtual void genNeuronUpdate(CodeStream &os, FileStreamCreator streamCreator, ModelSpecMerged &modelMerged,
                                 BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const final;
    virtual void genSynapseUpdate(CodeStream &os, FileStreamCreator streamCreator, ModelSpecMerged &modelMerged,
                                  BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const final;
    virtual void genCustomUpdate(CodeStream &os, FileStreamCreator streamCreator, ModelSpecMerged &modelMerged,
                                 BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const final;
    virtual void genInit(CodeStream &os, FileStreamCreator streamCreator, ModelSpecMerged &modelMerged,
                         BackendBase::MemorySpaces &memorySpaces, HostHandler preambleHandler) const final;

    virtual size_t getSynapticMatrixRowStride(const SynapseGroupInternal &sg) const final;

    virtual void genDefinitionsPreamble(CodeStream &os, const ModelSpecMerged &modelMerged) const final;
    virtual void genRunnerPreamble(CodeStream &os, const ModelSpecMerged &modelMerged) const final;
    virtual void genAllocateMemPreamble(CodeStream &os, const ModelSpecMerged &modelMerged) const final;
    virtual void genFreeMemPreamble(CodeStream &os, const ModelSpecMerged &modelMerged) const final;
    virtual void genStepTimeFinalisePreamble(CodeStream &os, const ModelSpecMerged &modelMerged) const final;

    // ---- runtime objects ---------------------------------------------------------------------------
    virtual std::unique_ptr<GeNN::Runtime::StateBase> createState(const Runtime::Runtime &runtime) const final;
    virtual std::unique_ptr<GeNN::Runtime::ArrayBase> createArray(const Type::ResolvedType &type, size_t count,
                                                                  VarLocation location, bool uninitialized) const final;
    virtual std::unique_ptr<GeNN::Runtime::ArrayBase> createPopulationRNG(size_t count) const final;

    virtual void genLazyVariableDynamicAllocation(CodeStream &os, const Type::ResolvedType &type, const std::string &name,
                                                  VarLocation loc, const std::string &countVarName) const final;
    virtual void genLazyVariableDynamicPush(CodeStream &os, const Type::ResolvedType &type, const std::string &name,
                                            VarLocation loc, const std::string &countVarName) const final;
    virtual void genLazyVariableDynamicPull(CodeStream &os, const Type::ResolvedType &type, const std::string &name,
                                            VarLocation loc, const std::string &countVarName) const final;
    virtual void genMergedDynamicVariablePush(CodeStream &os, const std::string &suffix, size_t mergedGroupIdx,
                                              const std::string &groupIdx, const std::string &fieldName,
                                              const std::string &egpName) const final;

    // ---- initialisation loop shapes ---------------------------------------------------------------
    virtual void genPopVariableInit(EnvironmentExternalBase &env, HandlerEnv handler) const final;
    virtual void genVariableInit(EnvironmentExternalBase &env, const std::string &count, const std::string &indexVarName,
                                 HandlerEnv handler) const final;
    virtual void genSparseSynapseVariableRowInit(EnvironmentExternalBase &env, HandlerEnv handler) const final;
    virtual void genDenseSynapseVariableRowInit(EnvironmentExternalBase &env, HandlerEnv handler) const final;
    virtual void genKernelSynapseVariableInit(EnvironmentExternalBase &env, SynapseInitGroupMerged &sg, HandlerEnv handler) const final;
    virtual void genKernelCustomUpdateVariableInit(EnvironmentExternalBase &env, CustomWUUpdateInitGroupMerged &cu, HandlerEnv handler) const final;

    virtual std::string getAtomicOperation(const std::string &lhsPointer, const std::string &rhsValue,
                                           const Type::ResolvedType &type, AtomicOperation op = AtomicOperation::ADD) const final;
    virtual std::string getRestrictKeyword() const final { return " __restrict__"; }

    virtual void genGlobalDeviceRNG(CodeStream &definitions, CodeStream &runner, CodeStream &allocations, CodeStream &free) const final;
    virtual void genTimer(CodeStream &definitions, CodeStream &runner, CodeStream &allocations, CodeStream &free,
                          CodeStream &stepTimeFinalise, const std::string &name, bool updateInStepTime) const final;
    virtual void genReturnFreeDeviceMemoryBytes(CodeStream &os) const final;
    virtual void genAssert(CodeStream &os, const std::string &condition) const final;

    // ---- build rules ---------------------------------------------------------------------------------
    virtual bool shouldUseNMakeBuildSystem() const final { return false; }
    virtual void genMakefilePreamble(std::ostream &os) const final;
    virtual void genMakefileLinkRule(std::ostream &os) const final;
    virtual void genMakefileCompileRule(std::ostream &os) const final;
    virtual void genNMakefilePreamble(std::ostream &os) const final;
    virtual void genNMakefileLinkRule(std::ostream &os) const final;
    virtual void genNMakefileCompileRule(std::ostream &os) const final;
    virtual void genMSBuildConfigProperties(std::ostream &os) const final;
    virtual void genMSBuildImportProps(std::ostream &os) const final;
    virtual void genMSBuildItemDefinitions(std::ostream &os) const final;
    virtual void genMSBuildCompileModule(const std::string &moduleName, std::ostream &os) const final;
    virtual void genMSBuildImportTarget(std::ostream &os) const final;

    // ---- predicates ------------------------------------------------------------------------------------
    virtual bool isArrayDeviceObjectRequired() const final { return true; }
    virtual bool isArrayHostObjectRequired() const final { return false; }
    virtual bool isGlobalHostRNGRequired(const ModelSpecInternal &model) const final;
    virtual bool isGlobalDeviceRNGRequired(const ModelSpecInternal &model) const final;
    virtual bool isPopulationRNGInitialisedOnDevice() const final { return true; }
    virtual bool isPostsynapticRemapRequired() const final { return true; }
    virtual bool isHostReductionRequired() const final { return false; }
    virtual size_t getDeviceMemoryBytes() const final;
    virtual MemorySpaces getMergedGroupMemorySpaces(const ModelSpecMerged &modelMerged) const final;
    virtual boost::uuids::detail::sha1::digest_type getHashDigest() const final;

private:
    unsigned int blockSize() const { return getPreferences<Preferences>().blockSize; }
    std::string includeDirectory() const;
};

//! Factory with the signature GeNN's front ends expect of a backend
//! (single_threaded_cpu/optimiser.h, backends/cuda/optimiser.h: createBackend)
Backend createBackend(const ModelSpecInternal &model, const filesystem::path &outputPath,
                      plog::Severity backendLevel, plog::IAppender *backendAppender,
                      const Preferences &preferences);
}   // namespace GeNN::CodeGenerator::B200
