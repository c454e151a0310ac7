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
    for f in ("cuda_tensor.hpp", "cuda_tensor.cpp", "cuda_optimizer.cpp", "cuda_program.cpp"):
        shutil.copy(os.path.join(REF, "src", "cuda", f), tree / "src" / "cuda" / f)
    mod.patch_tree(str(tree))
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


def test_integration_sources_name_every_entry_point_they_use():
    inc = open(os.path.join(ROOT, "saga_b200", "host", "e2e", "b200_create_optimizers.inc")).read()
    hdr = open(os.path.join(ROOT, "include", "b200opt.h")).read()
    for name in ("b200opt_layout", "b200opt_create", "b200opt_buffers", "b200opt_init_master",
                 "b200opt_flags"):
        assert name + "(" in inc and "int " + name + "(" in hdr
