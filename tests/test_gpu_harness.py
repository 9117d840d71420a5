"""The C++ harness executables (layoutCompare, layoutTest, netTest, stageBench) run, keep the reference's output format
("time:<ms> ms" lines that comparison/test.sh greps for) and pass their own host-side checks."""
import json
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "cudnntest_b200", "harness", "bin")


@pytest.fixture(scope="module", autouse=True)
def harness_built():
    """The executables are build products (git-ignored): compile them on the spot if this tree has none yet."""
    if not all(os.path.exists(os.path.join(BIN, e)) for e in ("layoutCompare", "layoutTest", "netTest", "stageBench")):
        import cudnntest_b200
        cudnntest_b200.build()


def run(exe, *args):
    p = subprocess.run([os.path.join(BIN, exe)] + list(args), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    return p.stdout


def summary(out):
    return json.loads([l for l in out.splitlines() if l.startswith("{")][-1])


@pytest.mark.parametrize("opt", [0, 1, 2])
@pytest.mark.parametrize("dtype", ["fp32", "fp32x3", "bf16"])
def test_layout_compare_ours(opt, dtype):
    out = run("layoutCompare", "batch=4", "opt=%d" % opt, "layer=6", "dtype=" + dtype, "iters=5")
    assert len(re.findall(r"time:[0-9.]+ ms", out)) == 5
    assert "moduleConv error" not in out
    s = summary(out)
    assert s["layout"] == ["NCHW", "NHWC", "CHWN"][opt] and s["max_err_sampled"] <= (1e-4 if dtype in ("fp32", "fp32x3") else 2e-2)


def test_layout_compare_cudnn_best():
    out = run("layoutCompare", "batch=4", "opt=8", "layer=6", "dtype=bf16", "iters=5")
    s = summary(out)
    assert s.get("unsupported") or ("cuDNN best" in s["what"] and s["max_err_sampled"] <= 2e-2)


def test_layout_compare_reference_cudnn_modes():
    for opt in (3, 6):
        out = run("layoutCompare", "batch=4", "opt=%d" % opt, "layer=6", "iters=3")
        s = summary(out)
        assert s.get("unsupported") or s["max_err_sampled"] <= 1e-3


@pytest.mark.parametrize("layout", ["NCHW", "NHWC", "CHWN"])
def test_layout_test_driver(layout, tmp_path):
    out = run("layoutTest", "8", "22", "128", "128", "layout=" + layout, "dir=" + str(tmp_path))
    assert re.search(r"time [0-9.]+ us\s+[0-9.]+ TFLOPS", out)
    assert "(ok)" in out and "moduleConv error" not in out
    assert os.path.getsize(os.path.join(str(tmp_path), "ConvModule_%s.bin" % layout)) == 8 * 128 * 22 * 22 * 4


@pytest.mark.parametrize("mode", [0, 1, 2, 4])
def test_net_test(mode):
    out = run("netTest", "set", "batch=4", "mode=%d" % mode, "dtype=bf16", "rounds=3")
    s = summary(out)
    if s.get("unsupported"):
        return
    assert len(re.findall(r"time:[0-9.]+ ms", out)) == 3 and s["images_per_s"] > 0


def test_net_test_separate_pool_and_hand_off():
    """fusepool=0 runs the block-end pooling as its own pass (the reference's sequencing); the classifier's verdict on
    the result must be the one of the fused run.  Mode 2 also exercises the CHWN -> NCHW FP32 hand-off of conv13."""
    tops = []
    for fuse in (1, 0):
        out = run("netTest", "set", "batch=2", "mode=2", "dtype=bf16", "rounds=1", "tail=1", "fusepool=%d" % fuse)
        s = summary(out)
        assert "classifier tail error" not in out and s["tail_top1_agree"] is True
        tops.append(re.findall(r"Batch \d+ Resulting weights from Softmax:(\d+)", out))
    assert tops[0] == tops[1] and len(tops[0]) == 2


@pytest.mark.parametrize("dtype,layout,wino", [("bf16", "nhwc", 4), ("fp32", "nchw", 4), ("tf32", "chwn", 2), ("fp32x3", "nhwc", 4)])
def test_stage_bench(dtype, layout, wino):
    """Per-stage micro-benchmark on the nine VGG-16 shapes: every staged pipeline passes its host-side check and the
    weighted sums (the reference's weightedSum line and the JSON summary) are printed."""
    out = run("stageBench", "batch=1", "dtype=" + dtype, "layout=" + layout, "wino=%d" % wino, "iters=2")
    assert len(re.findall(r"^case \d: .* valid=yes", out, flags=re.M)) == 9
    assert re.search(r"totalTime:[0-9.]+", out)
    s = summary(out)
    assert s["valid"] is True and s["weighted_us_vgg16"] > 0 and s["engine_weighted_us_vgg16"] > 0


@pytest.mark.parametrize("mode,dtype", [(1, "bf16"), (0, "fp32"), (2, "bf16"), (1, "fp32x3")])
def test_net_test_classifier_tail(mode, dtype):
    """netTest tail=1: fc14/fc15/fc16 + softmax + arg-max on the conv stack's output, checked by the harness against
    its host restatement (probabilities to 1e-4, same arg-max) for the first and the last image."""
    out = run("netTest", "set", "batch=3", "mode=%d" % mode, "dtype=" + dtype, "rounds=1", "tail=1")
    assert "classifier tail error" not in out
    assert len(re.findall(r"Batch \d+ Resulting weights from Softmax:\d+", out)) == 3
    s = summary(out)
    assert s["tail_max_abs_err"] <= 1e-4 and s["tail_top1_agree"] is True and s["tail_ms"] > 0
