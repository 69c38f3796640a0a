// pybind11 module `spncpy`: the same two classes the reference exports
// (python-interface/src/python-interface.cpp:19-64) on top of the compat C++ API.
// Kernel.execute additionally validates what the reference trusts blindly: the array is made
// C-contiguous, and a wrong element size or feature count raises instead of reading out of bounds.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "spnc-runtime.h"
#include "spnc.h"

namespace py = pybind11;
using spnc::Kernel;
using spnc::spn_compiler;

PYBIND11_MODULE(spncpy, m) {
  py::class_<Kernel>(m, "Kernel")
      .def(py::init<const std::string&, const std::string&, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                    unsigned, const std::string&>())
      .def("fileName", &Kernel::fileName)
      .def("kernelName", &Kernel::kernelName)
      .def("queryType", &Kernel::queryType)
      .def("target", &Kernel::target)
      .def("batchSize", &Kernel::batchSize)
      .def("numFeatures", &Kernel::numFeatures)
      .def("bytesPerFeature", &Kernel::bytesPerFeature)
      .def("numResults", &Kernel::numResults)
      .def("bytesPerResult", &Kernel::bytesPerResult)
      .def("dataType", &Kernel::dataType)
      .def("release", [](const Kernel& k) { spnc_rt::spn_runtime::instance().release(k); })
      .def("execute", [](const Kernel& kernel, long num_elements, py::array inputs) {
        if (num_elements < 0) throw std::runtime_error("RUNTIME ERROR: negative number of elements");
        py::array in = py::array::ensure(inputs, py::array::c_style);
        if (!in) throw std::runtime_error("RUNTIME ERROR: inputs are not convertible to a C-contiguous array");
        if ((size_t)in.itemsize() != kernel.bytesPerFeature())
          throw std::runtime_error("RUNTIME ERROR: input element size does not match the compiled feature type");
        if ((size_t)in.size() < (size_t)num_elements * kernel.numFeatures())
          throw std::runtime_error("RUNTIME ERROR: input array holds fewer than num_elements x numFeatures values");
        std::vector<py::ssize_t> shape{(py::ssize_t)num_elements};
        if (kernel.numResults() > 1) shape.push_back((py::ssize_t)kernel.numResults());
        py::array result(py::dtype(kernel.dataType()), shape);
        void* inPtr = const_cast<void*>(in.data());
        void* outPtr = result.mutable_data();
        {
          py::gil_scoped_release nogil;
          spnc_rt::spn_runtime::instance().execute(kernel, (size_t)num_elements, inPtr, outPtr);
        }
        return result;
      });

  py::class_<spn_compiler>(m, "SPNCompiler")
      .def(py::init())
      .def("compileQuery", [](const spn_compiler&, const std::string& inputFile, const spnc::options_t& options) {
        return spn_compiler::compileQuery(inputFile, options);
      })
      .def_static("isTargetSupported", [](const std::string& target) { return spn_compiler::isTargetSupported(target); })
      .def_static("isFeatureAvailable", [](const std::string& feature) { return spn_compiler::isFeatureSupported(feature); })
      .def_static("getHostArchitecture", []() { return spn_compiler::getHostArchitecture(); });
}
