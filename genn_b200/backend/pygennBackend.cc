// pybind11 module `b200_backend`: what PyGeNN needs of a backend module
// (pygenn/genn_model.py:674-685): a default-constructible `Preferences` whose attributes GeNNModel
// sets from its keyword arguments, and `_create_backend(model, output_path, backend_log_level,
// preferences)`.  Same shape as the reference's modules (pygenn/src/cudaBackend.cc:33-109,
// pygenn/src/singleThreadedCPUBackend.cc:22-52).  Registered with
// genn_b200.pygenn_plugin.register(), after which `GeNNModel(..., backend="b200")` selects it.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <plog/Appenders/ConsoleAppender.h>

#include "modelSpecInternal.h"
#include "path.h"

#include "backend.h"

using namespace GeNN;
using namespace GeNN::CodeGenerator::B200;

namespace
{
Backend createBackendForPython(const ModelSpecInternal &model, const std::string &outputPath,
                               plog::Severity backendLevel, const Preferences &preferences)
{
    auto *consoleAppender = new plog::ConsoleAppender<plog::TxtFormatter>;
    return createBackend(model, filesystem::path(outputPath), backendLevel, consoleAppender, preferences);
}
}

PYBIND11_MODULE(b200_backend, m)
{
    pybind11::module_::import("pygenn._genn");
    pybind11::module_::import("pygenn._runtime");

    pybind11::class_<Preferences, CodeGenerator::PreferencesBase>(m, "Preferences")
        .def(pybind11::init<>())
        .def_readwrite("device_id", &Preferences::deviceID)
        .def_readwrite("block_size", &Preferences::blockSize)
        .def_readwrite("include_path", &Preferences::includePath)
        .def_readwrite("nvcc_path", &Preferences::nvccPath);

    pybind11::class_<State, Runtime::StateBase>(m, "_Runtime");

    // PyGeNN builds __cuda_array_interface__ from this (pygenn/model_preprocessor.py:68-93)
    pybind11::class_<Array, Runtime::ArrayBase>(m, "_Array")
        .def_property_readonly("_device_pointer",
            [](Array &a)
            {
                return reinterpret_cast<uintptr_t>(a.getDevicePointer());
            });

    pybind11::class_<Backend, CodeGenerator::BackendBase>(m, "_Backend");

    m.def("_create_backend", &createBackendForPython, pybind11::return_value_policy::move);
}
