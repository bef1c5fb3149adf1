"""The reference's own Python wrappers must bind to the drop-in without a change.

`nectarml/cuda/tensor/conv.py` and `nectarml/cuda/tensor/matmul.py` of the reference call
`_nectarml.tensor.conv.*` / `_nectarml.tensor.matmul` positionally.  This test reads those call sites
from the reference checkout (when it is present on the machine), turns every argument expression into
the name of the quantity it passes (`stride[1]` -> stride_w, `out_grad._data_ptr` -> out_grad_ptr, ...)
and checks that the drop-in module `nectarml_b200._nectarml` takes exactly those parameters in exactly
that order -- so assigning the drop-in's functions to the attributes of the reference's extension module
leaves `nectarml.nn.Conv2d`, its autograd closures and the autocast flag working unchanged.
"""
import ast
import inspect
import os

import pytest

from nectarml_b200 import _nectarml as shim

REF = os.environ.get("NECTARML_REFERENCE", os.path.join(os.sep, "root", "reference"))  # the reference checkout, where there is one
CONV_PY = os.path.join(REF, "nectarml", "cuda", "tensor", "conv.py")
MATMUL_PY = os.path.join(REF, "nectarml", "cuda", "tensor", "matmul.py")

pytestmark = pytest.mark.skipif(not os.path.exists(CONV_PY), reason="reference checkout not on this machine")

AXIS = {"stride": "stride", "padding": "padding", "dilation": "dilation", "output_padding": "output_padding"}


def _meaning(node: ast.expr) -> str:
    """Name of the quantity an argument expression passes."""
    src = ast.unparse(node)
    if isinstance(node, ast.IfExp):  # `bias._data_ptr if bias is not None else 0`
        return _meaning(node.body)
    if isinstance(node, ast.Subscript) and isinstance(node.value, ast.Name) and node.value.id in AXIS:
        i = ast.literal_eval(node.slice)
        return f"{AXIS[node.value.id]}_{'hw'[i]}"
    if src.endswith("._data_ptr"):
        return src.split(".")[0] + "_ptr"
    if src.endswith(".size"):
        return src.split(".")[0] + "_size"
    if src.endswith(".numel()"):
        return src.split(".")[0]
    if src.endswith(".cuda"):
        return "dtype"
    if src.endswith(".shape"):
        return src.split(".")[0] + "_shape"
    return src


def _calls(path):
    tree = ast.parse(open(path).read())
    out = []
    for node in ast.walk(tree):
        if isinstance(node, ast.Call):
            name = ast.unparse(node.func)
            if name.startswith("_nectarml.tensor."):
                assert not node.keywords, f"{name} is called with keywords"
                out.append((name[len("_nectarml.tensor."):], [_meaning(a) for a in node.args]))
    return out


def _shim_params(dotted):
    obj = shim.tensor
    for part in dotted.split("."):
        obj = getattr(obj, part)
    return list(inspect.signature(obj).parameters)


def test_every_conv_call_site_binds_by_position_and_meaning():
    calls = _calls(CONV_PY)
    names = {c[0] for c in calls}
    assert {"conv.conv2d", "conv.conv_transpose2d", "conv.conv2d_backward_input", "conv.conv2d_backward_weight",
            "conv.conv_transpose2d_backward_input", "conv.conv_transpose2d_backward_weight", "conv.conv1d",
            "conv.conv_transpose1d"} <= names
    for name, passed in calls:
        want = _shim_params(name)
        assert len(passed) == len(want), (name, passed, want)
        for got, param in zip(passed, want):
            # the 1-D wrappers pass scalars named stride / padding / dilation / output_padding
            assert got == param or got.replace("out_grad", "out_grad") == param, (name, got, param)


def test_matmul_call_site_binds():
    (name, passed), = _calls(MATMUL_PY)
    assert name == "matmul"
    assert passed == ["a_ptr", "b_ptr", "a_shape", "b_shape", "dtype"] == _shim_params("matmul")


def test_free_path_and_dtype_values_match_the_reference():
    mem = open(os.path.join(REF, "nectarml", "cuda", "memory.py")).read()
    assert "_nectarml.free_cuda(" in mem
    assert list(inspect.signature(shim.free_cuda).parameters)[:1] == ["ptr"]
    dtype_h = open(os.path.join(REF, "nectarml", "csrc", "include", "common", "dtype.h")).read()
    body = dtype_h[dtype_h.index("enum class DType"):]
    order = [w.strip(" ,") for w in body[body.index("{") + 1:body.index("}")].split("\n") if w.strip()]
    order = [w.split("=")[0].split("//")[0].strip(" ,") for w in order]
    assert [o for o in order if o][:2] == ["Float32", "Float16"]
    assert int(shim.DType.Float32) == 0 and int(shim.DType.Float16) == 1
