"""Models written against the reference's layer API, run on this library and on the reference.

tests/cpp/layer_models.cu is one source compiled twice without a change: against dl_cuda_b200/src
(tests/cpp/libnative_models.so, the code under test) and against the reference's own headers
(oracle/_ref/libref_models.so, the checker).  oracle/_ref also holds the reference's char-LM example
(its src/examples_api.cu, unchanged) linked both ways.  The checker halves are built where the
reference checkout is present and travel as binaries; tests that need them skip when they are absent.

Tolerances: matrix products keep the reference's summation order and match bit for bit; layer norm,
softmax and bias gradients are summed in a different (parallel) order, so whole-layer results are
compared within 1e-4 of the tensor's scale (fp32, a few dozen chained reductions), and the training
loss of the character model within 2e-3 over the first 30 steps."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

from conftest import bits_equal, rel_err, rng_for

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
NATIVE = ROOT / "tests" / "cpp" / "libnative_models.so"
REFERENCE = ROOT / "oracle" / "_ref" / "libref_models.so"
CHAR_LM = {"native": ROOT / "oracle" / "_ref" / "char_lm_native", "ref": ROOT / "oracle" / "_ref" / "char_lm_ref"}

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)
_libs = {}


def load(which):
    if which not in _libs:
        path = NATIVE if which == "native" else REFERENCE
        if which == "native" and not path.exists():
            from dl_cuda_b200 import build
            build.build_cpp_tests()
        if not path.exists():
            pytest.skip(f"{path.name} not built (needs the reference checkout at build time)")
        lib = C.CDLL(str(path))
        lib.lm_transformer_run.argtypes = [C.c_int] * 7 + [_fp] * 6 + [C.c_int]
        lib.lm_linear_run.argtypes = [C.c_int] * 3 + [_fp] * 8
        lib.lm_softmax_run.argtypes = [C.c_int] * 2 + [_fp] * 4
        lib.lm_loss_run.argtypes = [C.c_int] * 3 + [_fp] * 4
        lib.lm_ce_ids_run.argtypes = [C.c_int] * 2 + [_ip] + [_fp] * 3
        lib.lm_schedule.argtypes = [C.c_float, C.c_float, C.c_int, C.c_int, _fp]
        lib.lm_schedule.restype = None
        lib.lm_char_lm_train.argtypes = [C.c_uint64] + [C.c_int] * 7 + [_ip, _ip, C.c_float, C.c_float, C.c_int,
                                                                      C.c_float, C.c_int, _fp, _fp, _fp, C.c_int,
                                                                      C.c_char_p]
        _libs[which] = lib
    return _libs[which]


def fp(a):
    return a.ctypes.data_as(_fp)


def transformer_run(which, layers, B, S, D, H, F, causal, x, dy):
    lib = load(which)
    n = B * S * D
    Fe = F if F > 0 else 4 * D
    per_layer = 4 * D * D + 2 * D * Fe + Fe + D + 4 * D
    total = layers * per_layer
    y, dx = np.empty(n, np.float32), np.empty(n, np.float32)
    params, grads = np.empty(total, np.float32), np.empty(total, np.float32)
    got = lib.lm_transformer_run(layers, B, S, D, H, F, int(causal), fp(x), fp(dy), fp(y), fp(dx), fp(params),
                                 fp(grads), total)
    assert got == total
    return y, dx, params, grads


def group_slices(layers, D, F):
    """(name, slice) of every parameter group in get_param_groups() order."""
    sizes = [("wq", D * D), ("wk", D * D), ("wv", D * D), ("wo", D * D), ("ff1_w", D * F), ("ff1_b", F),
             ("ff2_w", F * D), ("ff2_b", D), ("gamma1", D), ("beta1", D), ("gamma2", D), ("beta2", D)]
    out, at = [], 0
    for layer in range(layers):
        for name, size in sizes:
            out.append((f"layer{layer}.{name}", slice(at, at + size)))
            at += size
    return out


@pytest.mark.parametrize("layers,B,S,D,H,F,causal", [
    (1, 1, 8, 16, 2, 32, False),
    (1, 2, 16, 32, 4, 64, True),
    (3, 1, 64, 64, 4, 256, True),      # the char-LM example's model
    (2, 3, 20, 24, 3, 0, True),        # d_ff = 0 -> 4*d_model; sizes that are not multiples of the tiles
    (1, 32, 64, 64, 4, 256, False),    # batch 32 x seq 64: the char-LM shapes of the benchmark
])
def test_transformer_stack_matches_reference(layers, B, S, D, H, F, causal):
    g = rng_for(800, layers * 1000 + B * 100 + S)
    x = g.standard_normal(B * S * D).astype(np.float32)
    dy = g.standard_normal(B * S * D).astype(np.float32)
    Fe = F if F > 0 else 4 * D
    y, dx, params, grads = transformer_run("native", layers, B, S, D, H, F, causal, x, dy)
    assert np.isfinite(y).all() and np.isfinite(dx).all() and np.isfinite(grads).all()
    ry, rdx, rparams, rgrads = transformer_run("ref", layers, B, S, D, H, F, causal, x, dy)
    assert bits_equal(params, rparams), "std::mt19937(42) initialisation must agree bit for bit"
    assert rel_err(y, ry) < 1e-4
    assert rel_err(dx, rdx) < 1e-4
    for name, sl in group_slices(layers, D, Fe):
        assert rel_err(grads[sl], rgrads[sl]) < 2e-4, name


def test_transformer_layer_init_statistics():
    """Without the reference: weights ~ N(0, 2/fan_in), gammas 1, betas and biases 0, outputs normalised."""
    B, S, D, H, F = 2, 8, 32, 4, 64
    g = rng_for(801)
    x = g.standard_normal(B * S * D).astype(np.float32)
    y, dx, params, grads = transformer_run("native", 1, B, S, D, H, F, True, x, x)
    parts = dict((name.split(".")[1], params[sl]) for name, sl in group_slices(1, D, F))
    assert abs(parts["wq"].std() - np.sqrt(2 / D)) < 0.02 and abs(parts["ff2_w"].std() - np.sqrt(2 / F)) < 0.02
    assert np.all(parts["gamma1"] == 1) and np.all(parts["gamma2"] == 1)
    assert not parts["beta1"].any() and not parts["ff1_b"].any() and not parts["ff2_b"].any()
    rows = y.reshape(B * S, D)
    assert np.allclose(rows.mean(axis=1), 0, atol=1e-5) and np.allclose(rows.var(axis=1), 1, atol=1e-3)


@pytest.mark.parametrize("n,fin,fout", [(4, 2, 8), (64, 64, 30), (100, 33, 7), (4, 8, 1)])
def test_linear_layer_matches_reference(n, fin, fout):
    g = rng_for(810, n + fin)
    w = g.standard_normal(fin * fout).astype(np.float32)
    b = g.standard_normal(fout).astype(np.float32)
    x = g.standard_normal(n * fin).astype(np.float32)
    dy = g.standard_normal(n * fout).astype(np.float32)

    def run(which):
        out = [np.empty(k, np.float32) for k in (n * fout, n * fin, fin * fout, fout)]
        assert load(which).lm_linear_run(n, fin, fout, fp(w), fp(b), fp(x), fp(dy), *map(fp, out)) == 0
        return out

    y, dx, dw, db = run("native")
    want = x.reshape(n, fin).astype(np.float64) @ w.reshape(fin, fout) + b
    assert rel_err(y, want.ravel()) < 1e-5
    ry, rdx, rdw, rdb = run("ref")
    assert bits_equal(y, ry) and bits_equal(dx, rdx) and bits_equal(dw, rdw)
    assert rel_err(db, rdb) < 1e-5


def test_softmax_layer_and_losses_match_reference():
    g = rng_for(820)
    rows, width = 64, 30
    x = (2 * g.standard_normal(rows * width)).astype(np.float32)
    dy = g.standard_normal(rows * width).astype(np.float32)

    def softmax(which):
        y, dx = np.empty_like(x), np.empty_like(x)
        assert load(which).lm_softmax_run(rows, width, fp(x), fp(dy), fp(y), fp(dx)) == 0
        return y, dx

    y, dx = softmax("native")
    ry, rdx = softmax("ref")
    assert rel_err(y, ry) < 1e-6 and rel_err(dx, rdx) < 1e-5

    target = g.integers(0, width, rows).astype(np.int32)

    def ce(which):
        err, grad = np.empty(rows, np.float32), np.empty(rows * width, np.float32)
        assert load(which).lm_ce_ids_run(rows, width, target.ctypes.data_as(_ip), fp(ry), fp(err), fp(grad)) == 0
        return err, grad

    err, grad = ce("native")
    rerr, rgrad = ce("ref")
    assert bits_equal(grad, rgrad) and rel_err(err, rerr) < 1e-6

    for kind in range(4):
        classes = 5 if kind == 3 else 1
        n = 40
        if kind >= 2:
            yt = (g.random(n * classes) > 0.5).astype(np.float32)
            pred = g.random(n * classes).astype(np.float32)
        else:
            yt = g.standard_normal(n).astype(np.float32)
            pred = g.standard_normal(n).astype(np.float32)

        def loss(which):
            e, gr = np.empty(n, np.float32), np.empty(n * classes, np.float32)
            assert load(which).lm_loss_run(kind, n, classes, fp(yt), fp(pred), fp(e), fp(gr)) == 0
            return e, gr

        e, gr = loss("native")
        re_, rgr = loss("ref")
        assert rel_err(e, re_) < 1e-6 and rel_err(gr, rgr) < 1e-6, kind


def test_schedulers_match_reference_bit_for_bit():
    def schedule(which):
        lr = np.empty(120, np.float32)
        load(which).lm_schedule(3e-3, 1e-5, 50, 120, fp(lr))
        return lr

    lr = schedule("native")
    assert lr[0] == np.float32(3e-3) * np.float32(1 / 50) and lr[49] == np.float32(3e-3)
    assert np.all(np.diff(lr[:50]) > 0) and np.all(np.diff(lr[50:]) <= 0)
    assert bits_equal(lr, schedule("ref"))


def char_lm_train(which, seed, epochs, init=None, checkpoint=None):
    vocab, S, D, F, H, layers = 30, 64, 64, 256, 4, 3
    g = rng_for(830)
    # a repeating pattern of 23 tokens: the next token is predictable from the context
    stream = np.tile(g.integers(0, vocab, 23), (epochs * S + 1) // 23 + 1)[:epochs * S + 1].astype(np.int32)
    ids = np.stack([stream[e * S:(e + 1) * S] for e in range(epochs)]).copy()
    targets = np.stack([stream[e * S + 1:(e + 1) * S + 1] for e in range(epochs)]).copy()
    total = vocab * D + layers * (4 * D * D + 2 * D * F + F + D + 4 * D) + D * vocab + vocab
    p0 = np.empty(total, np.float32) if init is None else init.copy()
    losses, p1 = np.empty(epochs, np.float32), np.empty(total, np.float32)
    got = load(which).lm_char_lm_train(seed, vocab, S, D, F, H, layers, epochs, ids.ctypes.data_as(_ip),
                                       targets.ctypes.data_as(_ip), 3e-3, 1e-5, 5, 1.0, int(init is not None),
                                       fp(p0), fp(losses), fp(p1), total,
                                       str(checkpoint).encode() if checkpoint else None)
    assert got == total
    return p0, losses, p1


def test_char_lm_training_matches_reference(tmp_path):
    """Same start, 30 steps of clip + AdamW + warm-up/cosine: loss curve and parameters stay together."""
    epochs = 30
    init, rlosses, rfinal = char_lm_train("ref", 12345, epochs, checkpoint=tmp_path / "ref.bin")
    _, losses, final = char_lm_train("native", 12345, epochs, init=init, checkpoint=tmp_path / "native.bin")
    assert losses[0] == pytest.approx(rlosses[0], rel=1e-5)
    assert np.max(np.abs(losses - rlosses) / rlosses) < 2e-3
    assert losses[-1] < losses[0]
    assert rel_err(final, rfinal) < 5e-3
    a, b = (tmp_path / "native.bin").read_bytes(), (tmp_path / "ref.bin").read_bytes()
    assert len(a) == len(b) and a[:12] == b[:12]  # magic, version, group count
    sizes_a = np.frombuffer(a, np.int32)[3]
    assert sizes_a == np.frombuffer(b, np.int32)[3] == 30 * 64


def test_char_lm_training_learns_without_the_reference():
    """Runs everywhere the native library is built: the loss must fall on a repeating sequence."""
    _, losses, final = char_lm_train("native", 777, 40)
    assert np.isfinite(losses).all() and np.isfinite(final).all()
    assert 2.5 < losses[0] < 6.0  # about log(30) plus the spread of the untrained logits
    assert losses[-1] < 0.8 * losses[0]


def run_char_lm(which, path, epochs, load=False):
    binary = CHAR_LM[which]
    if not binary.exists():
        pytest.skip(f"{binary.name} not built (needs the reference checkout at build time)")
    args = [str(binary), epochs, 64, 1, 0, path] + (["load"] if load else [])
    res = subprocess.run(list(map(str, args)), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    loss = [float(m) for m in re.findall(r"Loss: ([0-9.]+)", res.stdout)]
    return res.stdout, np.array(loss)


def test_reference_char_lm_example_links_and_matches(tmp_path):
    """The reference's own examples_api.cu, compiled unchanged against this repository's headers."""
    # zero epochs: the checkpoint holds the initial weights (cuRAND embedding and head, mt19937 blocks)
    run_char_lm("native", tmp_path / "n0.bin", 0)
    run_char_lm("ref", tmp_path / "r0.bin", 0)
    assert (tmp_path / "n0.bin").read_bytes() == (tmp_path / "r0.bin").read_bytes(), "DLCU bytes at initialisation"
    # a short training run from the same initial weights
    out_n, loss_n = run_char_lm("native", tmp_path / "n.bin", 25)
    out_r, loss_r = run_char_lm("ref", tmp_path / "r.bin", 25)
    assert len(loss_n) == len(loss_r) == 25
    assert np.max(np.abs(loss_n - loss_r) / loss_r) < 5e-3
    lr_n = re.findall(r"LR: ([0-9.]+)", out_n)
    assert lr_n == re.findall(r"LR: ([0-9.]+)", out_r)
    a = np.frombuffer((tmp_path / "n.bin").read_bytes()[12:], np.float32)
    b = np.frombuffer((tmp_path / "r.bin").read_bytes()[12:], np.float32)
    assert a.size == b.size
    # each implementation reloads the other's checkpoint
    run_char_lm("native", tmp_path / "r.bin", 0, load=True)
    run_char_lm("ref", tmp_path / "n.bin", 0, load=True)


def test_reference_xor_example_matches():
    """run_xor of the reference's examples_api.cu (LinearLayer, ReLU, Sigmoid, Adam, binary cross entropy) on both
    header sets: the same loss log and final predictions."""
    logs = {}
    for which in ("native", "ref"):
        binary = CHAR_LM[which]
        if not binary.exists():
            pytest.skip(f"{binary.name} not built (needs the reference checkout at build time)")
        res = subprocess.run([str(binary), "xor", "1500", "100"], capture_output=True, text=True, timeout=300)
        if res.returncode == 2:
            pytest.skip(f"{binary.name} predates the xor mode: rebuild")
        assert res.returncode == 0, res.stdout + res.stderr
        bce = np.array([float(m) for m in re.findall(r"BCE: ([0-9.]+)", res.stdout)])
        pred = np.array([float(m) for m in re.findall(r"-> ([0-9.]+) \(expected", res.stdout)])
        assert bce.size == 15 and pred.size == 4
        logs[which] = (bce, pred)
    (bce_n, pred_n), (bce_r, pred_r) = logs["native"], logs["ref"]
    assert np.allclose(bce_n, bce_r, rtol=2e-3, atol=2e-5)
    assert np.allclose(pred_n, pred_r, atol=2e-3)
    # (with its default seed the reference's own run settles at 0.5 / 1 / 0.5 / 0 after 1500 epochs; what is
    # checked here is that both implementations follow the same trajectory, not how good that trajectory is)
    assert bce_n[-1] < bce_n[0]
