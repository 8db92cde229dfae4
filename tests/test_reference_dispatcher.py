"""The reference's own network-level dispatcher, unmodified, on top of this library.

`auto_tensorize_cuda` and `AutoTensorizeContext` are cut out of the reference checkout's
python/tvm/tensor_graph/core/auto_schedule/auto_schedule.py (:92-105, :351-433) at test time --
the file as a whole imports half of TVM -- and executed with `at` bound to
`amos_b200.auto_tensorize`.  That is the drop-in claim for this caller: its code does not change,
only what stands behind the `at.*` names.  Skipped where there is no reference checkout.
"""
import ast
import json
import os

import numpy as np
import pytest

from amos_b200 import _lib, tvm
from amos_b200 import auto_tensorize as at
import ops

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the checkout is looked for beside this repository unless AMOS_REFERENCE names it
REF_FILE = os.path.join(os.environ.get("AMOS_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference")),
                        "python/tvm/tensor_graph/core/auto_schedule/auto_schedule.py")
WANTED = ("auto_tensorize_cuda", "AutoTensorizeContext")


def _reference_dispatcher():
    """{name: object} for the two definitions, compiled from the reference's source text."""
    if not os.path.isfile(REF_FILE):
        pytest.skip("no reference checkout")
    with open(REF_FILE) as f:
        tree = ast.parse(f.read(), REF_FILE)
    picked = [n for n in tree.body
              if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in WANTED]
    assert sorted(n.name for n in picked) == sorted(WANTED)
    for n in picked:
        n.decorator_list = []  # `@tvm._ffi.register_func(...)`: registration in TVM's global table
    module = ast.Module(body=picked, type_ignores=[])
    scope = {"at": at, "os": os, "tvm": tvm}
    exec(compile(module, REF_FILE, "exec"), scope)
    return {name: scope[name] for name in WANTED}


class _Subgraph:
    def __init__(self, tensors, tag):
        self.root_ops = [t.op for t in tensors]
        self.tag = tag


def test_reference_dispatcher_plans_on_the_shimmed_names(built_lib, tmp_path, capsys):
    ref = _reference_dispatcher()
    A, B, C = ops.batch_gemm(12, 512, 512, 64)
    keep = tvm.te.create_schedule([C.op])
    (sch, args), = ref["auto_tensorize_cuda"](keep, [C], str(tmp_path / "bg.log"), 0).items()
    assert args == [A, B, C] and sch.plan.kind == _lib.OP_BATCHED_GEMM
    X = tvm.te.placeholder([8, 8], dtype="float16", name="X")
    Y = tvm.te.compute([8, 8], lambda i, j: X[i, j] + X[j, i], name="Y")
    keep2 = tvm.te.create_schedule([Y.op])
    assert ref["auto_tensorize_cuda"](keep2, [Y], str(tmp_path / "ew.log"), 0) == {keep2: []}

    Ctx = ref["AutoTensorizeContext"]
    mo = at.MeasureOptions(target="cuda", dev_id=0)
    sub = _Subgraph([C], "batch_gemm")
    assert Ctx.can_use("bg", str(tmp_path), sub, mo)
    assert not Ctx.can_use("ew", str(tmp_path), _Subgraph([Y], "ew"), mo)
    ctx = Ctx("bg", str(tmp_path), sub, mo)
    assert ctx.get_best_schedule() == (None, None, at.MAX_FLOAT)
    with open(ctx.log_name, "w") as f:
        print(json.dumps({"record": {"tile_n": [128, 0], "cta_pair": [1, 0]}, "value": 4000.0}),
              file=f)
    ctx2 = Ctx("bg", str(tmp_path), sub, mo)
    sch2, args2 = ctx2.auto_schedule(0)
    assert args2 == [A, B, C] and sch2.plan.tile_n == 128 and sch2.plan.cta_pair == 1
    assert abs(ctx2.get_best_schedule()[2] - 0.25) < 1e-9
    capsys.readouterr()


@pytest.mark.gpu
def test_reference_dispatcher_tunes_and_runs(oracle, tmp_path):
    """The reference's context tunes a linear layer through `at.find_optimized_parameters`, and the
    schedule it hands back builds into a module that computes the right numbers."""
    ref = _reference_dispatcher()
    A, B, C = ops.gemm_nt(384, 264, 200)
    mo = at.MeasureOptions(target="cuda", timeout=10, number=20, min_repeat_ms=10)
    ctx = ref["AutoTensorizeContext"]("fc", str(tmp_path), _Subgraph([C], "linear"), mo)
    sch, args = ctx.auto_schedule(4)
    assert ctx.total_trials == 4 and ctx.schedule_gen.has_entry()
    assert os.path.isfile(os.path.join(str(tmp_path), "at:fc.log"))
    assert 0 < ctx.get_best_schedule()[2] < 10
    func = tvm.build(sch, args, "cuda")
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, [int(x) for x in A.shape]).astype(np.float16)
    b = rng.uniform(-1, 1, [int(x) for x in B.shape]).astype(np.float16)
    c = tvm.nd.empty([int(x) for x in C.shape], C.dtype)
    func(tvm.nd.array(a), tvm.nd.array(b), c)
    assert oracle.rel_l2(c.asnumpy(), oracle.c_gemm(a, b, "te_llvm", trans_b=True)) <= 1e-3
