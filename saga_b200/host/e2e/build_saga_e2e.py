"""Builds the two end-to-end training binaries (needs the Saga checkout):

  _build/saga_e2e_ref    the reference library, unmodified (NCCL build),
                         + its own test/test_classifier.cpp + e2e_main.cpp
  _build/saga_cifar18_*  the same two library builds + e2e_cifar_resnet18.cpp
  _build/saga_parity_*   the same two library builds + e2e_parity.cpp
  _build/saga_e2e_b200   the same with the optimizer ops replaced by the
                         b200opt op: the library sources are copied to a
                         scratch directory outside this repository and
                         edited there by the small anchored rewrites below

(_build/ is this file's sibling directory.)  The checkout is the first argument,
else $SAGA_REFERENCE_DIR, else a directory "reference" beside this repository.

    python saga_b200/host/e2e/build_saga_e2e.py [/path/to/saga]

Nothing of the reference's source is stored in this repository; the rewrites
name only the identifiers they hang on.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", "..", ".."))
OUT = os.path.join(HERE, "_build")

LIB_SRCS = ["src/util.cpp", "src/tensor.cpp", "src/graph.cpp", "src/node.cpp", "src/engine.cpp",
            "src/ui/tui.cpp", "src/ui/nui.cpp", "src/pub.cpp",
            "src/cuda/cuda_common.cpp", "src/cuda/cuda_program.cpp", "src/cuda/cuda_analysis.cpp",
            "src/cuda/cuda_dnn.cpp", "src/cuda/cuda_optimizer.cpp", "src/cuda/cuda_tensor.cpp"]
KERNELS = "src/cuda/cuda_kernels.cu"
HARNESS = "test/test_classifier.cpp"

CXX = ["g++", "--std=c++17", "-O2", "-fPIC", "-mf16c", "-Wno-deprecated-declarations",
       "-Wno-terminate", "-I/usr/local/cuda/include"]
NVCC = ["/usr/local/cuda/bin/nvcc", "--std=c++17", "-O2", "-gencode",
        "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
LIBS = ["-L/usr/local/cuda/lib64", "-lcudart", "-lcudnn", "-lcublas", "-lpthread"]


def run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout[-3000:] + res.stderr[-6000:])
        raise SystemExit(1)


def rewrite(path, edits):
    text = open(path).read()
    for fn in edits:
        text = fn(text)
    open(path, "w").write(text)


def patch_tree(tree):
    """The b200opt integration, as edits anchored on identifiers of the Saga tree."""
    def storage_hpp(t):
        a = "CudaTensorStorageMemory(size_t size);"
        assert a in t
        return t.replace(a, a + "\n    CudaTensorStorageMemory(void *external, int)"
                                " : m_mem(external), m_external(true) {}\n"
                                "    bool m_external{false};", 1)

    def storage_cpp(t):
        a = "chkCuda(cudaFree(m_mem));"
        assert a in t
        t = t.replace(a, "if(!m_external)\n        " + a, 1)
        # host access to tensors in library-owned device memory goes through a staging copy
        b = "std::unique_ptr<TensorAccess>\nCudaTensor::access()"
        assert b in t
        t = t.replace(b, '#include <vector>\n#include <cstring>\n#include "b200_tensor_access.inc"\n\n' + b, 1)
        c = "return std::make_unique<CudaTensorAccess>(m_storage, m_desc, m_offset);"
        assert t.count(c) == 1
        return t.replace(c, "if(m_storage->m_memory && m_storage->m_memory->m_external)\n"
                            "        return std::make_unique<B200StagedTensorAccess>(m_storage, m_desc, "
                            "m_offset);\n    " + c, 1)

    def optimizer_cpp(t):
        start = t.index("CudaOps\nCudaProgram::create_optimizers()")
        end = t.rindex("}  // namespace saga")
        head = t[:start].replace('#include "cuda_kernels.hpp"',
                                 '#include "cuda_kernels.hpp"\n#include <mutex>\n#include <map>\n'
                                 '#include "cuda_aux.hpp"\n#include "b200_adam_op.hpp"', 1)
        return head + '#include "b200_create_optimizers.inc"\n\n' + t[end:]

    def program_cpp(t):
        # CudaProgram::step: the stream synchronise and the host policy block become
        # conditional on where the loss scale lives.  Scale on the host (default):
        # synchronise, fetch the flag sums, run the reference's own policy block.
        # Scale on the device: b200_pace() right behind the enqueue of the step's ops
        # keeps the host ONE step ahead of the device (it waits for the previous
        # step's end, so the batch callbacks that follow may touch the previous
        # step's buffers), and neither the synchronise nor the policy block runs.
        pos = t.index("m_mp_scaling *= 0.5")
        start = t.rindex("if(m_mp_enabled)", 0, pos)
        sync = "chkCuda(cudaStreamSynchronize(m_ctx->m_stream));"
        s0 = t.rindex(sync, 0, start)
        assert t[s0 + len(sync):start].strip() == ""
        t = (t[:s0] + "if(!b200_step_end(*this))\n        " + sync + "\n\n    b200_fill_aux(*this);\n\n    "
             + "if(m_mp_enabled && !m_b200_dscale)" + t[start + len("if(m_mp_enabled)"):])
        a = "runOps(m_ops, batch, m_pc.anomaly_detect);"
        assert t.count(a) == 1
        t = t.replace(a, a + "\n    b200_pace(*this);", 1)
        # buckets of the optimizer step are moved behind the backward ops they depend on
        b = "m_ops.insert(m_ops.end(), m_opt.begin(), m_opt.end());"
        assert t.count(b) == 1
        t = t.replace(b, b + "\n    b200_place_buckets(m_ops);", 1)
        a = "namespace saga {"
        i = t.index(a)
        return (t[:i] + a + "\nclass CudaProgram;\nvoid b200_fill_aux(CudaProgram &p);\n"
                "void b200_pace(CudaProgram &p);\nbool b200_step_end(CudaProgram &p);\n"
                "void b200_place_buckets(CudaOps &ops);\n"
                + t[i + len(a):])

    def common_hpp(t):
        a = "float m_mp_scaling{1};"
        assert t.count(a) == 1
        t = t.replace(a, a + "\n    const float *m_b200_dscale{nullptr};  // loss scale in device memory, or null", 1)
        b = "double getMPS(void) const override { return m_mp_scaling; }"
        assert t.count(b) == 1
        return t.replace(b, "double getMPS(void) const override;", 1)

    def kernels_cu(t):
        import re
        # one more parameter for the two loss-gradient kernel templates
        t, k = re.subn(r"(catclassifier_bwd\(int n, const T \*x, T \*dx, const L \*y, const L \*dy,\s*"
                       r"float \*loss, unsigned int channels, float scale)\)\s*\{",
                       r"\1, const float *dscale)\n{\n    if(dscale != nullptr)\n        scale = scale * *dscale;", t)
        assert k == 1
        t, k = re.subn(r"(deviceLossReduction\(const T \*A, const L \*B, T \*g, float scale, float \*out,\s*"
                       r"int N)\)\s*\{",
                       r"\1, const float *dscale)\n{\n    if(dscale != nullptr)\n        scale = scale * *dscale;", t)
        assert k == 1
        # the existing launchers pass null
        t, k = re.subn(r"loss, c, scale\);", "loss, c, scale, nullptr);", t)
        assert k == 2
        t, k = re.subn(r"x \+ o, dy \+ o, dx \+ o, scale, loss \+ i \* 4, c\);",
                       "x + o, dy + o, dx + o, scale, loss + i * 4, c, nullptr);", t)
        assert k == 3
        end = t.rindex("};  // namespace saga")
        return t[:end] + '#include "b200_loss_scale_kernels.inc"\n\n' + t[end:]

    def dnn_cpp(t):
        import re
        a = '#include "cuda_kernels.hpp"'
        assert t.count(a) == 1
        t = t.replace(a, a + '\n#include "b200_loss_scale.hpp"', 1)
        t, k = re.subn(r"\b(catclassifier_bwd_half_i32|loss_bwd_half_float|loss_bwd_half_half|"
                       r"loss_bwd_float_float)\(", r"b200_\1(", t)
        assert k == 4
        t, k = re.subn(r"scale \* p\.m_mp_scaling, p\.m_ctx->m_stream\)",
                       "scale, p.m_mp_scaling, p.m_b200_dscale, p.m_ctx->m_stream)", t)
        assert k == 4
        return t

    def node_cpp(t):
        # a defect of the tree that the integrated build trips over: the classifier's
        # per-sample loss output is declared with ONE element although its backward kernel
        # writes one float per sample; sized by the batch here
        a = 'makeTensor(Tensor::DataType::FLOAT, Dims({1, 1}), "loss");'
        assert t.count(a) == 1
        return t.replace(a, 'makeTensor(Tensor::DataType::FLOAT, Dims({x->m_dims[0], 1}), "loss");', 1)

    rewrite(os.path.join(tree, "src/node.cpp"), [node_cpp])
    rewrite(os.path.join(tree, "src/cuda/cuda_tensor.hpp"), [storage_hpp])
    rewrite(os.path.join(tree, "src/cuda/cuda_tensor.cpp"), [storage_cpp])
    rewrite(os.path.join(tree, "src/cuda/cuda_optimizer.cpp"), [optimizer_cpp])
    rewrite(os.path.join(tree, "src/cuda/cuda_program.cpp"), [program_cpp])
    rewrite(os.path.join(tree, "src/cuda/cuda_common.hpp"), [common_hpp])
    rewrite(os.path.join(tree, "src/cuda/cuda_kernels.cu"), [kernels_cu])
    rewrite(os.path.join(tree, "src/cuda/cuda_dnn.cpp"), [dnn_cpp])


def build_variant(ref, work, name, defines, extra_inc, extra_libs):
    objs = []
    inc = ["-I" + ref, "-I" + os.path.join(ref, "src")] + extra_inc
    procs = []
    for src in LIB_SRCS + [HARNESS]:
        obj = os.path.join(work, name + "_" + src.replace("/", "_") + ".o")
        objs.append(obj)
        procs.append(subprocess.Popen(CXX + defines + inc + ["-c", os.path.join(ref, src), "-o", obj],
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    kobj = os.path.join(work, name + "_kernels.o")
    run(NVCC + ["-I" + os.path.join(ref, "src", "cuda")] + extra_inc + ["-c", os.path.join(ref, KERNELS), "-o", kobj])
    mobj = os.path.join(work, name + "_main.o")
    run(CXX + defines + inc + ["-c", os.path.join(HERE, "e2e_main.cpp"), "-o", mobj])
    cobj = os.path.join(work, name + "_cifar.o")
    run(CXX + defines + inc + ["-c", os.path.join(HERE, "e2e_cifar_resnet18.cpp"), "-o", cobj])
    pobj = os.path.join(work, name + "_parity.o")
    run(CXX + defines + inc + ["-c", os.path.join(HERE, "e2e_parity.cpp"), "-o", pobj])
    for p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(out[-8000:])
            raise SystemExit(1)
    # link order follows the reference's Makefile: library objects, kernels, programs
    lib_objs, harness_obj = objs[:-1], objs[-1]
    exe = os.path.join(OUT, name)
    run(["g++", "-o", exe] + lib_objs + [kobj, mobj, harness_obj] + LIBS + extra_libs)
    # the CIFAR-variant ResNet-18 program uses the public API only
    exe2 = os.path.join(OUT, name.replace("saga_e2e", "saga_cifar18"))
    run(["g++", "-o", exe2] + lib_objs + [kobj, cobj] + LIBS + extra_libs)
    # the parity program: identical injected weights, scale log and trained weights on disk
    exe3 = os.path.join(OUT, name.replace("saga_e2e", "saga_parity"))
    run(["g++", "-o", exe3] + lib_objs + [kobj, pobj] + LIBS + extra_libs)
    return " ".join((exe, exe2, exe3))


def main():
    ref = (sys.argv[1] if len(sys.argv) > 1 else
           os.environ.get("SAGA_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference"))
    if not os.path.exists(os.path.join(ref, "saga.hpp")):
        print(f"Saga checkout not found at {ref}: keeping any prebuilt binaries")
        return
    os.makedirs(OUT, exist_ok=True)
    work = tempfile.mkdtemp(prefix="saga_e2e_")
    try:
        print(build_variant(ref, work, "saga_e2e_ref", ["-DHAVE_NCCL"], [], ["-lnccl"]))
        tree = os.path.join(work, "tree")
        shutil.copytree(ref, tree, ignore=shutil.ignore_patterns(".git", "build"))
        patch_tree(tree)
        libdir = os.path.join(ROOT, "saga_b200")
        print(build_variant(tree, work, "saga_e2e_b200", ["-DHAVE_B200OPT"],
                            ["-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(ROOT, "saga_b200", "host"),
                             "-I" + HERE],
                            ["-L" + libdir, "-lb200opt", "-Wl,-rpath,$ORIGIN/../../.."]))
    finally:
        shutil.rmtree(work, ignore_errors=True)


if __name__ == "__main__":
    main()
