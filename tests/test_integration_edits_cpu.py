"""The Saga-side integration is applied by anchored rewrites (build_saga_e2e.py);
when the Saga checkout is available, check on a scratch copy that every anchor
is found exactly where expected and that the rewritten files contain the hooks.
Skipped where the checkout is absent (nothing of it is stored in this repository)."""
import importlib.util
import os
import shutil

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("SAGA_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")


def _load():
    path = os.path.join(ROOT, "saga_b200", "host", "e2e", "build_saga_e2e.py")
    spec = importlib.util.spec_from_file_location("build_saga_e2e", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "saga.hpp")),
                    reason="Saga checkout not available")
def test_anchored_edits_apply_to_the_checkout(tmp_path):
    mod = _load()
    tree = tmp_path / "tree"
    os.makedirs(tree / "src" / "cuda")
    for f in ("cuda_tensor.hpp", "cuda_tensor.cpp", "cuda_optimizer.cpp", "cuda_program.cpp",
              "cuda_common.hpp", "cuda_kernels.cu", "cuda_dnn.cpp"):
        shutil.copy(os.path.join(REF, "src", "cuda", f), tree / "src" / "cuda" / f)
    shutil.copy(os.path.join(REF, "src", "node.cpp"), tree / "src" / "node.cpp")
    mod.patch_tree(str(tree))
    node = (tree / "src" / "node.cpp").read_text()
    assert 'Dims({x->m_dims[0], 1}), "loss")' in node and 'Dims({1, 1}), "loss")' not in node
    opt = (tree / "src" / "cuda" / "cuda_optimizer.cpp").read_text()
    assert '#include "b200_create_optimizers.inc"' in opt
    assert "CudaProgram::create_optimizers()" not in opt          # the original is gone
    assert "CudaProgram::create_optimizer(Tensor::DataType dt)" in opt  # the rest is untouched
    prog = (tree / "src" / "cuda" / "cuda_program.cpp").read_text()
    assert prog.count("b200_fill_aux(*this);") == 1
    assert prog.index("b200_fill_aux(*this);") < prog.index("m_mp_scaling *= 0.5")
    assert "bool m_external{false};" in (tree / "src" / "cuda" / "cuda_tensor.hpp").read_text()
    tensor_cpp = (tree / "src" / "cuda" / "cuda_tensor.cpp").read_text()
    assert "if(!m_external)" in tensor_cpp
    # host access to library-owned device memory is staged
    assert tensor_cpp.count('#include "b200_tensor_access.inc"') == 1
    assert tensor_cpp.index('#include "b200_tensor_access.inc"') < tensor_cpp.index("CudaTensor::access()")
    assert "std::make_unique<B200StagedTensorAccess>(m_storage, m_desc, m_offset)" in tensor_cpp
    assert tensor_cpp.count("std::make_unique<CudaTensorAccess>(m_storage, m_desc, m_offset)") == 1
    # CudaProgram::step: pacing hook behind the enqueue, the stream synchronise and the host
    # policy block only when the loss scale lives on the host
    assert prog.count("b200_pace(*this);") == 1
    assert prog.index("runOps(m_ops, batch") < prog.index("b200_pace(*this);") < \
        prog.index("run_batched_tensor_callbacks(m_pc.post_ops")
    assert "if(!b200_step_end(*this))\n        chkCuda(cudaStreamSynchronize(m_ctx->m_stream));" in prog
    assert "if(m_mp_enabled && !m_b200_dscale)" in prog
    # finalize: bucket ops are moved behind their anchors once the optimizer ops are appended
    assert prog.index("m_ops.insert(m_ops.end(), m_opt.begin(), m_opt.end());") < \
        prog.index("b200_place_buckets(m_ops);") < prog.index("reduceLiveranges(m_ops")
    common = (tree / "src" / "cuda" / "cuda_common.hpp").read_text()
    assert "const float *m_b200_dscale{nullptr};" in common
    assert "double getMPS(void) const override;" in common
    # the loss-gradient kernels take the device-resident scale; the old launchers pass null
    kern = (tree / "src" / "cuda" / "cuda_kernels.cu").read_text()
    assert kern.count("const float *dscale)") == 2 and kern.count("scale = scale * *dscale;") == 2
    assert kern.count("loss, c, scale, nullptr);") == 2
    assert kern.count("loss + i * 4, c, nullptr);") == 3
    assert kern.count('#include "b200_loss_scale_kernels.inc"') == 1
    dnn = (tree / "src" / "cuda" / "cuda_dnn.cpp").read_text()
    assert dnn.count("scale, p.m_mp_scaling, p.m_b200_dscale, p.m_ctx->m_stream)") == 4
    assert "scale * p.m_mp_scaling" not in dnn
    for name in ("catclassifier_bwd_half_i32", "loss_bwd_half_float", "loss_bwd_half_half",
                 "loss_bwd_float_float"):
        assert dnn.count("b200_" + name + "(") == 1


def test_integration_sources_name_every_entry_point_they_use():
    inc = open(os.path.join(ROOT, "saga_b200", "host", "e2e", "b200_create_optimizers.inc")).read()
    hdr = open(os.path.join(ROOT, "include", "b200opt.h")).read()
    shim = open(os.path.join(ROOT, "saga_b200", "host", "b200_adam_op.hpp")).read()
    for name in ("b200opt_layout", "b200opt_create", "b200opt_buffers", "b200opt_init_master",
                 "b200opt_flags"):
        assert name + "(" in inc and "int " + name + "(" in hdr
    for name in ("b200opt_step", "b200opt_step_begin", "b200opt_step_bucket",
                 "b200opt_device_scale_enable", "b200opt_device_scale_ptr",
                 "b200opt_step_device_scale", "b200opt_device_scale_read",
                 "b200opt_device_scale_peek"):
        assert name + "(" in shim and "int " + name + "(" in hdr
