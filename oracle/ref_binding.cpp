// Binding used only by oracle/build_ref.py: exposes build_codebook of the reference's own
// src/huffman.cpp (compiled where it lies, unmodified) so that the C restatement in
// kvc_oracle.c can be checked against it.  Test infrastructure, never part of the product.
#include <torch/extension.h>
#include <huffman.h>

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("build_codebook", &build_codebook, "reference build_codebook (src/huffman.cpp:99-157)");
}
