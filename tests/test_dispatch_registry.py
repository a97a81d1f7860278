"""The dispatch registry of the host mirror (rai_b200/tensor.py) against the reference's own list of rules
(register_backend!, rai-core/src/dispatch.rs:41-157): every op of that list is either a registered rule for `Cuda`, a
view or transfer that the Tensor class does itself without a kernel rule, a 1-D form lowered onto its 2-D rule, or
one of the two random generators, which are the only ops left out.  Pure host logic: no GPU needed."""
import pytest

from rai_b200 import _lib, tensor
from rai_b200.device import Cuda

REFERENCE_OPS = """Abs Add Arange ArgMax ArgMin AvgPool1d AvgPool2d Broadcast Concatenate Conv1d Conv2d ConvTranspose1d
ConvTranspose2d Cos Div Equal Erf Exp FromArray Full Gather Greater GreaterEqual IndexAdd IndexSelect Less LessEqual Log
Log10 Log2 LogSoftmax MatMul MaxPool1d MaxPool2d Maximum Minimum Mul Narrow Negative Normal NotEqual Permute Powf Random
ReduceMax ReduceMin ReduceSum Reshape Rsqrt ScatterAdd Sign Sin Softmax Sqrt Square Sub Tanh ToContiguous ToDType ToDevice
Transpose UpsampleNearest1d UpsampleNearest2d Where""".split()

VIEWS_AND_TRANSFERS = {"Broadcast": "broadcast_to", "Narrow": "narrow", "Permute": "permute", "Reshape": "reshape",
                       "Transpose": "transpose", "FromArray": "from_array", "ToDevice": "as_vec"}
LOWERED_TO_2D = {"Conv1d": "conv1d", "ConvTranspose1d": "conv_transpose1d", "MaxPool1d": "max_pool1d",
                 "AvgPool1d": "avg_pool1d", "UpsampleNearest1d": "upsample_nearest1d"}
LEFT_OUT = {"Random", "Normal"}


def test_every_reference_rule_is_accounted_for():
    registered = {op for (dev, op) in tensor._RULES if dev is Cuda}
    for op in REFERENCE_OPS:
        if op in registered:
            continue
        method = VIEWS_AND_TRANSFERS.get(op) or LOWERED_TO_2D.get(op)
        if method:
            assert hasattr(tensor.Tensor, method), f"{op}: Tensor.{method} is missing"
            continue
        assert op in LEFT_OUT, f"{op} of the reference's rule list has neither a rule nor a Tensor method"
    assert not (LEFT_OUT & registered)


def test_a_missing_rule_is_unimplemented_and_register_overwrites():
    class OtherDevice:
        pass
    with pytest.raises(_lib.RaiB200Error) as e:            # Error::Unimplemented{op, device}, eval.rs:40-43
        tensor.eval_rule(OtherDevice(), "Add")
    assert e.value.code == -7
    first, second = (lambda *a: 1), (lambda *a: 2)
    tensor.register(OtherDevice, "Add", first)
    assert tensor.eval_rule(OtherDevice(), "Add") is first
    tensor.register(OtherDevice, "Add", second)             # dispatch::register overwrites, dispatch.rs:191-204
    assert tensor.eval_rule(OtherDevice(), "Add") is second
    del tensor._RULES[(OtherDevice, "Add")]
