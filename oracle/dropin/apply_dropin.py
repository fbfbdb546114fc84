#!/usr/bin/env python
"""TEST INFRASTRUCTURE. Applies the drop-in edits of INTEGRATION.md to a TEMPORARY copy of the
reference tree, so that the reference's own Tensor::matmul / Tensor::backward can be shown to run on
Device::cuda(0) tensors through libtfb.so.

    apply_dropin.py <reference root> <empty output directory>

Nothing of the reference is stored in this repository: the script copies the reference's files into the
output directory (outside the repository) and inserts OUR lines after or before anchor lines it finds
by regular expression. Four files are touched:

  cuda/CudaKernelRegistry.hpp       + MatmulFn / MatmulBackwardFn / FillFn and their register_* functions
  tensor/Tensor.cpp                 + the three function pointers, their setters, and a CUDA branch in
                                      Tensor::matmul before the "CPU only" check
  autograd/ops/MatmulBackward.hpp   + a CUDA branch in apply(): one call instead of two transposes and two products
  autograd/TensorAutograd.cpp       + the ones-fill of Tensor::backward on the device for CUDA tensors
"""
import os
import re
import shutil
import sys


def edit(path, anchor, text, where="after", count=1):
    src = open(path).read()
    m = list(re.finditer(anchor, src, flags=re.M))
    if len(m) < count:
        raise SystemExit(f"{path}: anchor {anchor!r} not found")
    m = m[count - 1]
    pos = m.end() if where == "after" else m.start()
    open(path, "w").write(src[:pos] + text + src[pos:])


def main():
    ref, out = sys.argv[1], sys.argv[2]
    for d in ("tensor", "autograd", "nn", "cuda", "third_party/mdspan", "third_party/doctest"):
        shutil.copytree(os.path.join(ref, d), os.path.join(out, d), dirs_exist_ok=True)

    # 1. registry slots
    edit(os.path.join(out, "cuda/CudaKernelRegistry.hpp"), r"^void register_current_stream\(void\* stream\);\n", """
// --- libtfb drop-in: the dense-contraction slots -------------------------------------------------
using MatmulFn = void (*)(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, Dtype in,
                          Dtype out, void* stream);
using MatmulBackwardFn = void (*)(const void* dC, const void* a, const void* b, void* dA, void* dB, int64_t M,
                                  int64_t N, int64_t K, Dtype dtype, void* stream);
using FillFn = void (*)(void* dst, int64_t n, float value, void* stream);
void register_cuda_matmul(MatmulFn fn);
void register_cuda_matmul_backward(MatmulBackwardFn fn);
void register_cuda_fill(FillFn fn);
MatmulBackwardFn registered_cuda_matmul_backward();
FillFn registered_cuda_fill();
void* registered_current_stream();
""")

    # 2. Tensor.cpp: pointers, setters, CUDA branch
    tensor_cpp = os.path.join(out, "tensor/Tensor.cpp")
    edit(tensor_cpp, r"^void\* g_current_stream = nullptr;\n", """MatmulFn g_cuda_matmul = nullptr;                    // libtfb drop-in
MatmulBackwardFn g_cuda_matmul_backward = nullptr;   // libtfb drop-in
FillFn g_cuda_fill = nullptr;                        // libtfb drop-in
""")
    edit(tensor_cpp, r"^void register_current_stream\(void\* stream\) \{[^\n]*\}\n", """void register_cuda_matmul(MatmulFn fn) { g_cuda_matmul = fn; }
void register_cuda_matmul_backward(MatmulBackwardFn fn) { g_cuda_matmul_backward = fn; }
void register_cuda_fill(FillFn fn) { g_cuda_fill = fn; }
MatmulBackwardFn registered_cuda_matmul_backward() { return g_cuda_matmul_backward; }
FillFn registered_cuda_fill() { return g_cuda_fill; }
void* registered_current_stream() { return g_current_stream; }
""")
    # the branch goes right before the device check of Tensor::matmul (the shape checks above it stay)
    edit(tensor_cpp, r"^    if \(this->device\(\)\.type != DeviceType::CPU \|\| other\.device\(\)\.type != DeviceType::CPU\) \{\n"
                     r"        throw std::invalid_argument\(\"Tensor::matmul: CPU only", """    if (this->device().type == DeviceType::CUDA && other.device().type == DeviceType::CUDA) {   // libtfb drop-in
        if (other.device() != this->device()) throw std::invalid_argument("Tensor::matmul: device mismatch");
        if (dtype() != other.dtype()) throw std::invalid_argument("Tensor::matmul: dtype mismatch");
        if (g_cuda_matmul == nullptr) throw std::runtime_error("CUDA matmul kernel not registered");
        Tensor cuda_out = Tensor::empty(Shape{shape_[0], other.shape_[1]}, dtype(), device());
        g_cuda_matmul(this->data(), other.data(), cuda_out.data(), shape_[0], other.shape_[1], shape_[1], dtype(), dtype(),
                      g_current_stream);
        if (g_wire_matmul != nullptr) g_wire_matmul(cuda_out, *this, other);
        return cuda_out;
    }
""", where="before")

    # 3. MatmulBackward::apply
    mb = os.path.join(out, "autograd/ops/MatmulBackward.hpp")
    edit(mb, r"^#include \"tensor/Tensor\.hpp\"\n", "#include \"cuda/CudaKernelRegistry.hpp\"   // libtfb drop-in\n")
    edit(mb, r"^        const Tensor& b = b_\.unpack\(\);\n", """        if (a.device().type == DeviceType::CUDA) {   // libtfb drop-in: no transposes, one call
            auto fn = registered_cuda_matmul_backward();
            if (fn == nullptr) throw std::runtime_error("CUDA matmul backward kernel not registered");
            Tensor cuda_ga = Tensor::empty(a.shape(), a.dtype(), a.device());
            Tensor cuda_gb = Tensor::empty(b.shape(), b.dtype(), b.device());
            fn(grads[0].data(), a.data(), b.data(), cuda_ga.data(), cuda_gb.data(), a.shape()[0], b.shape()[1],
               a.shape()[1], a.dtype(), registered_current_stream());
            return {std::move(cuda_ga), std::move(cuda_gb)};
        }
""")

    # 4. Tensor::backward: ones on the device
    ta = os.path.join(out, "autograd/TensorAutograd.cpp")
    edit(ta, r"^#include \"autograd/TensorAutograd\.hpp\"\n|^#include \"tensor/Tensor\.hpp\"\n",
         "#include \"cuda/CudaKernelRegistry.hpp\"   // libtfb drop-in\n")
    edit(ta, r"^    if \(dtype\(\) == Dtype::Float32 && grad\.numel\(\) > 0\) \{\n", """    if (device().type == DeviceType::CUDA) {   // libtfb drop-in: the root gradient is filled on the device
        auto fill = registered_cuda_fill();
        if (fill == nullptr) throw std::runtime_error("CUDA fill kernel not registered");
        fill(grad.data(), grad.numel(), 1.0f, registered_current_stream());
    } else
""", where="before")
    print("drop-in applied in", out)


if __name__ == "__main__":
    main()
