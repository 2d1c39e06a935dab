// Driver that runs a network description on the UNMODIFIED reference
// (GeNN 5.4.0 libgenn + its single_threaded_cpu backend, both compiled from
// the reference tree by oracle/Makefile.ref).  It is the ground truth the C
// restatement in oracle/genn_oracle.c and the CUDA kernels are pinned to.
//
// Test infrastructure only: the product never links, loads or executes it.
//
//   ref_driver <spec.txt> <work_dir> <out_dir> [generate]
//
// Compiled a second time with -DGENN_B200_BACKEND (-> b200_driver) the same
// program selects the B200 code-generation backend (genn_b200/backend) instead
// of the CPU one: identical model description, identical GeNN runtime, only the
// backend differs.  That binary is how the tests drive the plug-in.  With a
// fourth argument `generate` the program stops after generating and compiling
// the model's code (needs no GPU).
//
// The spec is the line-based text format written by genn_b200.netspec
// (one item per line, whitespace-separated tokens, arrays as raw
// little-endian files relative to the spec's directory).  Only the public
// model-building API of the reference is used (modelSpec.h:373-530), then
// code generation (generateModules.h:29), the generated Makefile and the
// reference's own Runtime (runtime.h:288-330) exactly as its generator
// front-end does.
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include <plog/Appenders/ConsoleAppender.h>
#include "path.h"

#include "logging.h"
#include "modelSpecInternal.h"
#include "code_generator/generateMakefile.h"
#include "code_generator/generateModules.h"
#include "code_generator/modelSpecMerged.h"
#include "runtime/runtime.h"
#ifdef GENN_B200_BACKEND
#include "../genn_b200/backend/backend.h"
#else
#include "optimiser.h"
#endif

using namespace GeNN;
#ifdef GENN_B200_BACKEND
namespace SelectedBackend = GeNN::CodeGenerator::B200;
#else
namespace CPU = GeNN::CodeGenerator::SingleThreadedCPU;
#endif

// Models that are NOT among GeNN's built-in ones: their code strings reach a backend only
// through the transpiler and the group emitters, which is what a drop-in backend must handle.
//
// Quadratic integrate-and-fire neuron with an adaptation current
class AdaptiveQIF : public NeuronModels::Base
{
public:
    DECLARE_SNIPPET(AdaptiveQIF);

    SET_SIM_CODE(
        "const scalar drive = (k * (V - Vrest) * (V - Vcrit)) + Isyn + Ioffset - W;\n"
        "V += dt * drive / C;\n"
        "W += dt * ((a * (V - Vrest)) - W) / tauW;\n");
    SET_THRESHOLD_CONDITION_CODE("V >= Vpeak");
    SET_RESET_CODE(
        "V = Vreset;\n"
        "W += b;\n");
    SET_PARAMS({"C", "k", "Vrest", "Vcrit", "Vpeak", "Vreset", "a", "b", "tauW", "Ioffset"});
    SET_VARS({{"V", "scalar"}, {"W", "scalar"}});
    SET_NEEDS_AUTO_REFRACTORY(false);
};
IMPLEMENT_SNIPPET(AdaptiveQIF);

// Pulse coupling whose weight is scaled by a parameter and saturates
class ScaledSaturatingPulse : public WeightUpdateModels::Base
{
public:
    DECLARE_SNIPPET(ScaledSaturatingPulse);

    SET_PARAMS({"gScale", "gMax"});
    SET_VARS({{"g", "scalar", VarAccess::READ_ONLY}});
    SET_PRE_SPIKE_SYN_CODE("addToPost(fmin(g * gScale, gMax));\n");
};
IMPLEMENT_SNIPPET(ScaledSaturatingPulse);

namespace
{
std::string g_specDir;

template<typename T>
std::vector<T> readFile(const std::string &name, size_t expect = 0)
{
    const std::string path = g_specDir + "/" + name;
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if(!f) throw std::runtime_error("cannot open " + path);
    const size_t bytes = (size_t)f.tellg();
    f.seekg(0);
    std::vector<T> v(bytes / sizeof(T));
    f.read(reinterpret_cast<char*>(v.data()), bytes);
    if(expect && v.size() != expect) {
        throw std::runtime_error(path + ": expected " + std::to_string(expect) + " elements, found " + std::to_string(v.size()));
    }
    return v;
}

template<typename T>
void writeFile(const std::string &path, const T *data, size_t n)
{
    std::ofstream f(path, std::ios::binary);
    f.write(reinterpret_cast<const char*>(data), n * sizeof(T));
}

struct PopSpec
{
    std::string name, kind;
    unsigned int n = 0;
    std::vector<double> p;
    std::vector<std::string> files;
    NeuronGroup *ng = nullptr;
};

struct CSSpec
{
    std::string name, pop, kind;
    std::vector<double> p;
};

struct SynSpec
{
    std::string name, matrix, src, trg, wum, psm;
    std::vector<double> wumP, psmP;
    unsigned int axDelay = 0, maxDenDelay = 0, maxConn = 0, backDelay = 0;
    std::string fRowLength, fInd, fG, fD, fGp;
    SynapseGroup *sg = nullptr;
};

std::vector<std::string> tokens(const std::string &line)
{
    std::istringstream ss(line);
    std::vector<std::string> t;
    std::string s;
    while(ss >> s) t.push_back(s);
    return t;
}
}   // anonymous namespace

int main(int argc, char *argv[])
{
    try {
        if(argc != 4 && argc != 5) {
            std::cerr << "usage: ref_driver <spec.txt> <work_dir> <out_dir> [generate]" << std::endl;
            return EXIT_FAILURE;
        }
        const bool generateOnly = (argc == 5) && (std::string(argv[4]) == "generate");
        const std::string specPath = argv[1];
        const filesystem::path workDir(argv[2]);
        const std::string outDir = argv[3];
        const size_t slash = specPath.find_last_of('/');
        g_specDir = (slash == std::string::npos) ? "." : specPath.substr(0, slash);

        // ---- parse -----------------------------------------------------------
        std::string modelName = "net";
        double dt = 0.1;
        unsigned int seed = 0, steps = 0, dumpEvery = 0;
        bool fusePSM = false, narrowInd = false, timing = true;
        std::vector<PopSpec> pops;
        std::vector<CSSpec> css;
        std::vector<SynSpec> syns;
        {
            std::ifstream f(specPath);
            if(!f) throw std::runtime_error("cannot open " + specPath);
            std::string line;
            while(std::getline(f, line)) {
                const auto t = tokens(line);
                if(t.empty() || t[0][0] == '#') continue;
                if(t[0] == "name") modelName = t[1];
                else if(t[0] == "dt") dt = std::stod(t[1]);
                else if(t[0] == "seed") seed = (unsigned int)std::stoul(t[1]);
                else if(t[0] == "steps") steps = (unsigned int)std::stoul(t[1]);
                else if(t[0] == "dump_every") dumpEvery = (unsigned int)std::stoul(t[1]);
                else if(t[0] == "fuse_psm") fusePSM = (t[1] == "1");
                else if(t[0] == "narrow_ind") narrowInd = (t[1] == "1");
                else if(t[0] == "timing") timing = (t[1] == "1");       // per-kernel timers (they synchronise every step)
                else if(t[0] == "pop") {
                    PopSpec p;
                    p.name = t[1]; p.n = (unsigned int)std::stoul(t[2]); p.kind = t[3];
                    size_t i = 4;
                    const size_t numP = (p.kind == "LIF") ? 7 : (p.kind == "IZH") ? 4 : (p.kind == "POISSON") ? 1
                                        : (p.kind == "AQIF") ? 10 : 0;
                    for(size_t k = 0; k < numP; k++) p.p.push_back(std::stod(t.at(i++)));
                    for(; i < t.size(); i++) p.files.push_back(t[i]);
                    pops.push_back(p);
                }
                else if(t[0] == "cs") {
                    CSSpec c;
                    c.name = t[1]; c.pop = t[2]; c.kind = t[3];
                    for(size_t i = 4; i < t.size(); i++) c.p.push_back(std::stod(t[i]));
                    css.push_back(c);
                }
                else if(t[0] == "syn") {
                    SynSpec s;
                    s.name = t[1]; s.matrix = t[2]; s.src = t[3]; s.trg = t[4];
                    size_t i = 5;
                    while(i < t.size()) {
                        const std::string k = t[i++];
                        if(k == "wum") {
                            s.wum = t.at(i++);
                            const size_t n = (s.wum == "CONST") ? 1 : (s.wum == "STDP") ? 6 : (s.wum == "SCALED") ? 2 : 0;
                            for(size_t j = 0; j < n; j++) s.wumP.push_back(std::stod(t.at(i++)));
                        }
                        else if(k == "psm") {
                            s.psm = t.at(i++);
                            const size_t n = (s.psm == "EXPCURR") ? 1 : (s.psm == "EXPCOND") ? 2 : 0;
                            for(size_t j = 0; j < n; j++) s.psmP.push_back(std::stod(t.at(i++)));
                        }
                        else if(k == "axdelay") s.axDelay = (unsigned int)std::stoul(t.at(i++));
                        else if(k == "backdelay") s.backDelay = (unsigned int)std::stoul(t.at(i++));
                        else if(k == "maxdendelay") s.maxDenDelay = (unsigned int)std::stoul(t.at(i++));
                        else if(k == "maxconn") s.maxConn = (unsigned int)std::stoul(t.at(i++));
                        else if(k == "rowlength") s.fRowLength = t.at(i++);
                        else if(k == "ind") s.fInd = t.at(i++);
                        else if(k == "g") s.fG = t.at(i++);
                        else if(k == "d") s.fD = t.at(i++);
                        else if(k == "gp") s.fGp = t.at(i++);
                        else throw std::runtime_error("unknown syn key " + k);
                    }
                    syns.push_back(s);
                }
                else throw std::runtime_error("unknown spec item " + t[0]);
            }
        }

        // ---- build the model through the reference's public API ---------------
        plog::ConsoleAppender<plog::TxtFormatter> consoleAppender;
#ifdef GENN_B200_BACKEND
        SelectedBackend::Preferences prefs;
#else
        CPU::Preferences prefs;
#endif
        Logging::init(plog::warning, plog::warning, plog::warning, plog::warning,
                      &consoleAppender, &consoleAppender, &consoleAppender, &consoleAppender);

        ModelSpecInternal model;
        model.setName(modelName);
        model.setDT(dt);
        model.setSeed(seed);
        model.setTimingEnabled(timing);
        model.setFusePostsynapticModels(fusePSM);
        model.setDefaultNarrowSparseIndEnabled(narrowInd);

        std::map<std::string, PopSpec*> popByName;
        for(auto &p : pops) {
            if(p.kind == "LIF") {
                ParamValues pv{{"C", p.p[0]}, {"TauM", p.p[1]}, {"Vrest", p.p[2]}, {"Vreset", p.p[3]},
                               {"Vthresh", p.p[4]}, {"Ioffset", p.p[5]}, {"TauRefrac", p.p[6]}};
                VarValues vv{{"V", uninitialisedVar()}, {"RefracTime", uninitialisedVar()}};
                p.ng = model.addNeuronPopulation<NeuronModels::LIF>(p.name, p.n, pv, vv);
            }
            else if(p.kind == "IZH") {
                ParamValues pv{{"a", p.p[0]}, {"b", p.p[1]}, {"c", p.p[2]}, {"d", p.p[3]}};
                VarValues vv{{"V", uninitialisedVar()}, {"U", uninitialisedVar()}};
                p.ng = model.addNeuronPopulation<NeuronModels::Izhikevich>(p.name, p.n, pv, vv);
            }
            else if(p.kind == "AQIF") {
                ParamValues pv{{"C", p.p[0]}, {"k", p.p[1]}, {"Vrest", p.p[2]}, {"Vcrit", p.p[3]}, {"Vpeak", p.p[4]},
                               {"Vreset", p.p[5]}, {"a", p.p[6]}, {"b", p.p[7]}, {"tauW", p.p[8]}, {"Ioffset", p.p[9]}};
                VarValues vv{{"V", uninitialisedVar()}, {"W", uninitialisedVar()}};
                p.ng = model.addNeuronPopulation<AdaptiveQIF>(p.name, p.n, pv, vv);
            }
            else if(p.kind == "SSA") {
                VarValues vv{{"startSpike", uninitialisedVar()}, {"endSpike", uninitialisedVar()}};
                p.ng = model.addNeuronPopulation<NeuronModels::SpikeSourceArray>(p.name, p.n, {}, vv);
            }
            else if(p.kind == "POISSON") {
                ParamValues pv{{"rate", p.p[0]}};
                VarValues vv{{"timeStepToSpike", 0.0}};
                p.ng = model.addNeuronPopulation<NeuronModels::Poisson>(p.name, p.n, pv, vv);
            }
            else throw std::runtime_error("unknown neuron model " + p.kind);
            p.ng->setSpikeRecordingEnabled(true);
            popByName[p.name] = &p;
        }
        for(auto &c : css) {
            NeuronGroup *ng = popByName.at(c.pop)->ng;
            if(c.kind == "POISSONEXP") {
                model.addCurrentSource<CurrentSourceModels::PoissonExp>(
                    c.name, ng, {{"weight", c.p[0]}, {"tauSyn", c.p[1]}, {"rate", c.p[2]}}, {{"current", 0.0}});
            }
            else if(c.kind == "DC") {
                model.addCurrentSource<CurrentSourceModels::DC>(c.name, ng, {{"amp", c.p[0]}}, {});
            }
            else throw std::runtime_error("unknown current source " + c.kind);
        }
        for(auto &s : syns) {
            NeuronGroup *src = popByName.at(s.src)->ng;
            NeuronGroup *trg = popByName.at(s.trg)->ng;
            const SynapseMatrixType mt = (s.matrix == "SPARSE") ? SynapseMatrixType::SPARSE
                : (s.matrix == "BITMASK") ? SynapseMatrixType::BITMASK : SynapseMatrixType::DENSE;

            PostsynapticModels::Init psm = (s.psm == "EXPCURR")
                ? initPostsynaptic<PostsynapticModels::ExpCurr>({{"tau", s.psmP[0]}})
                : (s.psm == "EXPCOND")
                    ? initPostsynaptic<PostsynapticModels::ExpCond>({{"tau", s.psmP[0]}, {"E", s.psmP[1]}}, {},
                                                                    {{"V", createVarRef(trg, "V")}})
                    : initPostsynaptic<PostsynapticModels::DeltaCurr>();

            if(s.wum == "STATIC") {
                s.sg = model.addSynapsePopulation(s.name, mt, src, trg,
                    initWeightUpdate<WeightUpdateModels::StaticPulse>({}, {{"g", uninitialisedVar()}}), psm);
            }
            else if(s.wum == "CONST") {
                s.sg = model.addSynapsePopulation(s.name, mt, src, trg,
                    initWeightUpdate<WeightUpdateModels::StaticPulseConstantWeight>({{"g", s.wumP[0]}}), psm);
            }
            else if(s.wum == "DENDELAY") {
                s.sg = model.addSynapsePopulation(s.name, mt, src, trg,
                    initWeightUpdate<WeightUpdateModels::StaticPulseDendriticDelay>(
                        {}, {{"g", uninitialisedVar()}, {"d", uninitialisedVar()}}), psm);
            }
            else if(s.wum == "SCALED") {
                s.sg = model.addSynapsePopulation(s.name, mt, src, trg,
                    initWeightUpdate<ScaledSaturatingPulse>({{"gScale", s.wumP[0]}, {"gMax", s.wumP[1]}},
                                                            {{"g", uninitialisedVar()}}), psm);
            }
            else if(s.wum == "STDP") {
                s.sg = model.addSynapsePopulation(s.name, mt, src, trg,
                    initWeightUpdate<WeightUpdateModels::STDP>(
                        {{"tauPlus", s.wumP[0]}, {"tauMinus", s.wumP[1]}, {"Aplus", s.wumP[2]},
                         {"Aminus", s.wumP[3]}, {"Wmin", s.wumP[4]}, {"Wmax", s.wumP[5]}},
                        {{"g", uninitialisedVar()}}), psm);
            }
            else throw std::runtime_error("unknown weight update model " + s.wum);

            if(s.maxConn) s.sg->setMaxConnections(s.maxConn);
            if(s.axDelay) s.sg->setAxonalDelaySteps(s.axDelay);
            if(s.backDelay) s.sg->setBackPropDelaySteps(s.backDelay);
            if(s.maxDenDelay) s.sg->setMaxDendriticDelayTimesteps(s.maxDenDelay);
        }

        model.finalise();

        // ---- generate, build, load -------------------------------------------
        filesystem::create_directory(workDir);
        const filesystem::path outputPath = workDir / (model.getName() + "_CODE");
        filesystem::create_directory(outputPath);
#ifdef GENN_B200_BACKEND
        auto backend = SelectedBackend::createBackend(model, outputPath, plog::warning, &consoleAppender, prefs);
#else
        auto backend = CPU::Optimiser::createBackend(model, outputPath, plog::warning, &consoleAppender, prefs);
#endif
        CodeGenerator::ModelSpecMerged modelMerged(backend, model);
        const auto moduleNames = CodeGenerator::generateAll(modelMerged, backend, outputPath, false);
        {
            std::ofstream makefile((outputPath / "Makefile").str());
            CodeGenerator::generateMakefile(makefile, backend, moduleNames);
        }
        // IEEE-strict -O3: the generated Makefile compiles with $(CXX) and adds no
        // optimisation flag of its own unless optimize_code (-ffast-math) is set
        const char *envCXX = std::getenv("REF_CXX");
        const std::string cxx = envCXX ? envCXX : "/usr/bin/g++ -O3";
        const std::string buildCommand = "make -s -C \"" + outputPath.str() + "\" -j 8 CXX=\"" + cxx + "\"";
        if(system(buildCommand.c_str()) != 0) {
            throw std::runtime_error("building generated code failed: " + buildCommand);
        }
        if(generateOnly) {
            std::cout << "generated and compiled " << outputPath.str() << std::endl;
            return EXIT_SUCCESS;
        }

        Runtime::Runtime runtime(workDir, modelMerged, backend);
        runtime.allocate(steps);
        runtime.initialize();

        // ---- host-supplied state and connectivity -----------------------------
        for(auto &p : pops) {
            if(p.kind == "LIF" || p.kind == "IZH" || p.kind == "AQIF") {
                const char *v1 = (p.kind == "LIF") ? "RefracTime" : (p.kind == "IZH") ? "U" : "W";
                auto V = readFile<float>(p.files.at(0), p.n);
                auto R = readFile<float>(p.files.at(1), p.n);
                std::copy(V.begin(), V.end(), runtime.getArray(*p.ng, "V")->getHostPointer<float>());
                std::copy(R.begin(), R.end(), runtime.getArray(*p.ng, v1)->getHostPointer<float>());
            }
            else if(p.kind == "SSA") {
                auto st = readFile<uint32_t>(p.files.at(0), p.n);
                auto en = readFile<uint32_t>(p.files.at(1), p.n);
                auto times = readFile<float>(p.files.at(2));
                std::copy(st.begin(), st.end(), runtime.getArray(*p.ng, "startSpike")->getHostPointer<uint32_t>());
                std::copy(en.begin(), en.end(), runtime.getArray(*p.ng, "endSpike")->getHostPointer<uint32_t>());
                runtime.allocateArray(*p.ng, "spikeTimes", std::max<size_t>(1, times.size()));
                auto *arr = runtime.getArray(*p.ng, "spikeTimes");
                std::copy(times.begin(), times.end(), arr->getHostPointer<float>());
                arr->pushToDevice();
            }
        }
        for(auto &s : syns) {
            const unsigned int numPre = popByName.at(s.src)->n;
            const unsigned int numPost = popByName.at(s.trg)->n;
            if(s.matrix == "SPARSE") {
                const size_t stride = s.maxConn;
                auto rl = readFile<uint32_t>(s.fRowLength, numPre);
                auto ind = readFile<uint32_t>(s.fInd, (size_t)numPre * stride);
                std::copy(rl.begin(), rl.end(), runtime.getArray(*s.sg, "rowLength")->getHostPointer<uint32_t>());
                auto *indArr = runtime.getArray(*s.sg, "ind");
                const size_t indSize = indArr->getType().getValue().size;
                for(size_t i = 0; i < ind.size(); i++) {
                    if(indSize == 1) indArr->getHostPointer<uint8_t>()[i] = (uint8_t)ind[i];
                    else if(indSize == 2) indArr->getHostPointer<uint16_t>()[i] = (uint16_t)ind[i];
                    else indArr->getHostPointer<uint32_t>()[i] = ind[i];
                }
                if(!s.fG.empty()) {
                    auto g = readFile<float>(s.fG, (size_t)numPre * stride);
                    std::copy(g.begin(), g.end(), runtime.getArray(*s.sg, "g")->getHostPointer<float>());
                }
                if(!s.fD.empty()) {
                    auto d = readFile<uint8_t>(s.fD, (size_t)numPre * stride);
                    std::copy(d.begin(), d.end(), runtime.getArray(*s.sg, "d")->getHostPointer<uint8_t>());
                }
            }
            else if(s.matrix == "BITMASK") {
                auto gp = readFile<uint32_t>(s.fGp);
                auto *arr = runtime.getArray(*s.sg, "gp");
                if(gp.size() != arr->getCount()) throw std::runtime_error("gp size mismatch for " + s.name);
                std::copy(gp.begin(), gp.end(), arr->getHostPointer<uint32_t>());
            }
            else {
                if(!s.fG.empty()) {
                    auto g = readFile<float>(s.fG, (size_t)numPre * numPost);
                    std::copy(g.begin(), g.end(), runtime.getArray(*s.sg, "g")->getHostPointer<float>());
                }
            }
        }
        runtime.initializeSparse();

        // ---- simulate ----------------------------------------------------------
        // a device backend's arrays are pulled before they are read (no-op on the CPU backend)
        auto pulled = [](Runtime::ArrayBase *arr)
        {
            if((arr->getLocation() & VarLocationAttribute::HOST) && (arr->getLocation() & VarLocationAttribute::DEVICE)) {
                arr->pullFromDevice();
            }
            return arr;
        };
        auto dump = [&](unsigned int step)
        {
            const std::string suffix = "_" + std::to_string(step) + ".bin";
            for(auto &p : pops) {
                if(p.kind == "LIF" || p.kind == "IZH" || p.kind == "AQIF") {
                    const char *v1 = (p.kind == "LIF") ? "RefracTime" : (p.kind == "IZH") ? "U" : "W";
                    writeFile(outDir + "/V_" + p.name + suffix, pulled(runtime.getArray(*p.ng, "V"))->getHostPointer<float>(), p.n);
                    writeFile(outDir + "/" + v1 + "_" + p.name + suffix, pulled(runtime.getArray(*p.ng, v1))->getHostPointer<float>(), p.n);
                }
            }
            for(auto &s : syns) {
                // with fused postsynaptic models only one group per fused set owns outPost
                try {
                    auto *arr = pulled(runtime.getArray(*s.sg, "outPost"));
                    writeFile(outDir + "/outPost_" + s.name + suffix, arr->getHostPointer<float>(), arr->getCount());
                }
                catch(const std::out_of_range&) {}
                try {
                    auto *arr = pulled(runtime.getArray(*s.sg, "denDelay"));
                    writeFile(outDir + "/denDelay_" + s.name + suffix, arr->getHostPointer<float>(), arr->getCount());
                }
                catch(const std::out_of_range&) {}
                if(s.wum == "STDP") {
                    auto *arr = pulled(runtime.getArray(*s.sg, "g"));
                    writeFile(outDir + "/g_" + s.name + suffix, arr->getHostPointer<float>(), arr->getCount());
                }
            }
        };

        double loopSeconds = 0.0;
        for(unsigned int i = 0; i < steps; i++) {
            const auto t0 = std::chrono::steady_clock::now();
            runtime.stepTime();
            loopSeconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if(dumpEvery && ((i + 1) % dumpEvery) == 0) dump(i + 1);
        }
        if(!dumpEvery || (steps % dumpEvery) != 0) dump(steps);

        // ---- spikes: (step, id) pairs per population ---------------------------
        runtime.pullRecordingBuffersFromDevice();
        for(auto &p : pops) {
            const auto rec = runtime.getRecordedSpikes(*p.ng);
            const auto &times = rec.at(0).first;
            const auto &ids = rec.at(0).second;
            std::vector<uint32_t> out(2 * times.size());
            for(size_t k = 0; k < times.size(); k++) {
                out[2 * k] = (uint32_t)std::llround(times[k] / dt);
                out[2 * k + 1] = ids[k];
            }
            writeFile(outDir + "/spikes_" + p.name + ".bin", out.data(), out.size());
        }
        {
            std::ofstream f(outDir + "/timing.txt");
            f << "loop_seconds " << loopSeconds << "\n"
              << "neuron_update_seconds " << runtime.getNeuronUpdateTime() << "\n"
              << "presynaptic_update_seconds " << runtime.getPresynapticUpdateTime() << "\n"
              << "postsynaptic_update_seconds " << runtime.getPostsynapticUpdateTime() << "\n"
              << "steps " << steps << "\n";
        }
        return EXIT_SUCCESS;
    }
    catch(const std::exception &e) {
        std::cerr << "ref_driver: " << e.what() << std::endl;
        return EXIT_FAILURE;
    }
}
