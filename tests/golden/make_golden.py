"""Writes tests/golden/*.npz: small seeded inputs with the outputs of the REFERENCE's own,
unmodified CUDA kernels (through oracle/_ref/libref_shim.so).  Needs a CUDA device and the
prebuilt shim; run once as

    python tests/golden/make_golden.py [--out DIR]

The fixtures pin the CPU oracle (tests/test_oracle_golden.py, no GPU needed) and the CUDA
kernels (tests/test_golden_gpu.py).  Gradient fixtures of the embedding use values that are
exact in fp32 under any summation order, because the reference adds them with atomicAdd.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import ref  # noqa: E402


def rng(seed):
    return np.random.Generator(np.random.Philox(key=seed))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def layernorm_case(rows, d, seed):
    g = rng(seed)
    a = g.standard_normal((rows, d)).astype(np.float32)
    b = g.standard_normal((rows, d)).astype(np.float32)
    gamma = g.uniform(0.5, 1.5, d).astype(np.float32)
    beta = (0.1 * g.standard_normal(d)).astype(np.float32)
    dy_a = g.standard_normal((rows, d)).astype(np.float32)
    dy_b = g.standard_normal((rows, d)).astype(np.float32)
    s = ref.residual_add(dev(a), dev(b))
    y, xhat, inv_std = ref.ln_fwd(s, dev(gamma), dev(beta), 1e-5)
    dsum = ref.residual_add(dev(dy_a), dev(dy_b))
    dx, dgamma, dbeta = ref.ln_bwd(dsum, xhat, inv_std, dev(gamma))
    return dict(a=a, b=b, gamma=gamma, beta=beta, eps=np.float32(1e-5), dy_a=dy_a, dy_b=dy_b, y=host(y),
                xhat=host(xhat), inv_std=host(inv_std), dx=host(dx), dgamma=host(dgamma), dbeta=host(dbeta))


def activation_case(rows, cols, seed):
    g = rng(seed)
    x = (2.0 * g.standard_normal((rows, cols))).astype(np.float32)
    x.ravel()[:8] = [0.0, -0.0, 1.0, -1.0, 20.0, -20.0, 88.0, -88.0]
    bias = (0.1 * g.standard_normal(cols)).astype(np.float32)
    dy = g.standard_normal((rows, cols)).astype(np.float32)
    out = dict(x=x, bias=bias, dy=dy)
    pre = ref.bias_add(dev(x), dev(bias))
    out["pre"] = host(pre)
    for kind, name in ((0, "relu"), (1, "sigmoid"), (2, "tanh"), (3, "gelu")):
        y, cache = ref.act_fwd(kind, pre)
        out[f"{name}_y"] = host(y)
        out[f"{name}_dx"] = host(ref.act_bwd(kind, dev(dy), cache))
    out["dbias_of_dy"] = host(ref.bias_grad(dev(dy)))
    return out


def embedding_case(vocab, d, batch, seq, seed):
    g = rng(seed)
    n = batch * seq
    table = (0.02 * g.standard_normal((vocab, d))).astype(np.float32)
    ids = g.integers(0, vocab, n).astype(np.int32)
    ids[: n // 4] = ids[0]  # a long run of duplicates
    dy = (g.integers(-8, 9, (n, d)) / 4.0).astype(np.float32)  # exact sums in any order
    pe = ref.pe_table(seq, d)
    gathered = ref.embed_fwd(dev(table), dev(ids))
    out = ref.pe_add(gathered.view(batch, seq, d), pe.cuda())
    grad = ref.embed_bwd(dev(dy), dev(ids), vocab)
    return dict(table=table, ids=ids, dy=dy, seq=np.int32(seq), pe=pe.numpy(), gathered=host(gathered),
                out=host(out).reshape(n, d), grad=host(grad))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent))
    args = ap.parse_args()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out / "layernorm_37x100.npz", **layernorm_case(37, 100, 11))
    np.savez_compressed(out / "layernorm_16x1024.npz", **layernorm_case(16, 1024, 12))
    np.savez_compressed(out / "layernorm_5x3.npz", **layernorm_case(5, 3, 13))
    np.savez_compressed(out / "activation_9x40.npz", **activation_case(9, 40, 21))
    np.savez_compressed(out / "embedding_v50_d12.npz", **embedding_case(50, 12, 4, 16, 31))
    # the reference's own known-answer test of the embedding layer, through its class
    table = np.arange(15, dtype=np.float32).reshape(5, 3)
    ids = np.array([1, 3, 1, 4], np.int32)
    dout = np.repeat(np.arange(1, 5, dtype=np.float32)[:, None], 3, axis=1)
    o, gr = ref.embedding_layer_run(table, ids, dout)
    init = ref.embedding_init(3, 5, 3, 4)  # the second layer this process builds: seed 3 + 9973*2
    np.savez_compressed(out / "embedding_layer_known_answer.npz", table=table, ids=ids, dout=dout, out=o, grad=gr,
                        curand_table_seed3=init)
    sgd_p = rng(41).standard_normal(257).astype(np.float32)
    sgd_g = rng(42).standard_normal(257).astype(np.float32)
    np.savez_compressed(out / "sgd_257.npz", p=sgd_p, g=sgd_g, lr=np.float32(0.05),
                        out=host(ref.sgd(dev(sgd_p), dev(sgd_g), 0.05)))
    print("wrote", sorted(p.name for p in out.glob("*.npz")))


if __name__ == "__main__":
    main()
