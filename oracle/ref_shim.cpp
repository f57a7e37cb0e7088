// TEST INFRASTRUCTURE ONLY -- never linked into or loaded by the product library.
//
// A small pybind11 module that is compiled *together with* the reference's own
// Metadata translation unit (sparseconvnet/SCN/Metadata/Metadata.cpp, pulled in
// from the read-only reference checkout by -I at build time; nothing is copied
// into this repository) and exposes the rulebooks that the reference keeps
// private to C++ (sparseconvnet/SCN/pybind.cpp:12-33 binds none of them).
//
// The Metadata_<D> Python objects are created by the reference's own SCN module;
// pybind11 shares the class registration between extension modules of one
// interpreter, so the functions below accept those objects directly.
//
// Every rulebook is returned as a list (one entry per filter offset / sample) of
// int32 tensors holding the flat (input_row, output_row) pairs exactly as the
// reference produced them (sparseconvnet/SCN/Metadata/Metadata.h:35).

#define ENABLE_OPENMP YES
#include <omp.h>
#include <torch/extension.h>

#include "Metadata/Metadata.cpp"

namespace {

std::vector<at::Tensor> rulebook_to_tensors(const RuleBook &rb) {
  std::vector<at::Tensor> out;
  out.reserve(rb.size());
  for (auto const &r : rb) {
    auto t = torch::empty({(long)r.size()}, at::kInt);
    if (!r.empty())
      std::memcpy(t.data_ptr<int>(), r.data(), r.size() * sizeof(Int));
    out.push_back(t);
  }
  return out;
}

// Metadata<D>::getSubmanifoldRuleBook  (Metadata.cpp:437-451)
template <Int D>
std::vector<at::Tensor> submanifold_rulebook(Metadata<D> &m, at::Tensor spatialSize,
                                             at::Tensor filterSize) {
  return rulebook_to_tensors(m.getSubmanifoldRuleBook(spatialSize, filterSize, true));
}

// Metadata<D>::getRuleBook  (Metadata.cpp:492-518); creates the coarse grid as a side effect
template <Int D>
std::vector<at::Tensor> strided_rulebook(Metadata<D> &m, at::Tensor inputSize,
                                         at::Tensor outputSize, at::Tensor filterSize,
                                         at::Tensor filterStride) {
  return rulebook_to_tensors(
      m.getRuleBook(inputSize, outputSize, filterSize, filterStride, true));
}

// Metadata<D>::getSparseToDenseRuleBook  (Metadata.cpp:476-491)
template <Int D>
std::vector<at::Tensor> sparse_to_dense_rulebook(Metadata<D> &m, at::Tensor spatialSize) {
  return rulebook_to_tensors(m.getSparseToDenseRuleBook(spatialSize, true));
}

// Metadata<D>::inputLayerRuleBook  (Metadata.h:59, filled by IOLayersRules.h:18-121)
template <Int D> std::vector<at::Tensor> input_layer_rulebook(Metadata<D> &m) {
  return rulebook_to_tensors(m.inputLayerRuleBook);
}

template <Int D> long n_active(Metadata<D> &m, at::Tensor spatialSize) {
  return m.getNActive(spatialSize);
}

template <Int D> void bind_dim(py::module &m) {
  m.def("submanifold_rulebook", &submanifold_rulebook<D>);
  m.def("strided_rulebook", &strided_rulebook<D>);
  m.def("sparse_to_dense_rulebook", &sparse_to_dense_rulebook<D>);
  m.def("input_layer_rulebook", &input_layer_rulebook<D>);
  m.def("n_active", &n_active<D>);
}

} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  bind_dim<1>(m);
  bind_dim<2>(m);
  bind_dim<3>(m);
  bind_dim<4>(m);
}
