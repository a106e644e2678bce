"""Generate the golden fixtures in this directory from the reference's own CPU code.

Run once, in a container where the reference checkout is mounted:

    TORCH_DEVICE_BACKEND_AUTOLOAD=0 python tests/golden/make_golden.py /path/to/reference

It imports the reference's pure-CPU modules (``tests/paged_attention_reference.py``,
``tests/fp64_reference.py``, ``tests/decoder_cpu_reference.py``) and, for reference
functions that live in device smoke scripts which cannot be imported without the device
module, compiles just that one function from the script's syntax tree.  Inputs and the
reference's outputs are written to ``*.npz`` (bf16 payloads as uint16 bit patterns).  The
fixtures travel with the repository; the reference does not.
"""
from __future__ import annotations

import ast
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def lift(path: str, name: str, env: dict):
    """Compile one top-level function of a reference script without running the script."""
    tree = ast.parse(open(path, encoding="utf-8").read())
    node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
    scope = dict(env)
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), scope)
    return scope[name]


def attention_cases(ref_tests):
    import paged_attention_reference as par
    from fp64_reference import direct_bf16

    cases = [
        # name, heads, kv_heads, d, slots, requests, context, rows(list of (request, position))
        ("gqa4_d64", 8, 2, 64, 96, 3, 24, [(0, 0), (0, 1), (1, 23), (2, 7), (2, 8), (1, 12)]),
        ("gqa8_d128", 8, 1, 128, 160, 2, 70, [(0, 69), (1, 33), (1, 0), (0, 64)]),
        ("mha_d64", 4, 4, 64, 80, 2, 36, [(0, 35), (1, 17), (1, 18)]),
    ]
    out = {}
    gen = torch.Generator().manual_seed(20261101)
    for name, heads, kv_heads, d, slots, n_req, context, rows in cases:
        perm = torch.randperm(slots - 1, generator=gen)[: n_req * context] + 1
        mapping = perm.reshape(n_req, context).to(torch.int32)
        requests = torch.tensor([r for r, _ in rows], dtype=torch.int64)
        positions = torch.tensor([p for _, p in rows], dtype=torch.int64)
        q = torch.randn(len(rows), heads * d, generator=gen).to(torch.bfloat16)
        kp = torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16)
        vp = torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16)
        scale = torch.tensor(1.0 / math.sqrt(d), dtype=torch.float32).item()
        env = {"torch": torch, "HEADS": heads, "KV_HEADS": kv_heads, "DIM": d,
               "Q_WIDTH": heads * d, "SCALE_FP32": scale}
        unrounded = lift(os.path.join(ref_tests, "paged_attention_smoke.py"), "expected_unrounded", env)
        args = (q, kp, vp, requests, positions, mapping)
        rec = {
            "heads": heads, "kv_heads": kv_heads, "head_dim": d, "scale": np.float64(scale),
            "mapping": mapping.numpy(), "requests": requests.numpy(), "positions": positions.numpy(),
            "q": bits(q), "key_pool": bits(kp), "value_pool": bits(vp),
            "unrounded32": unrounded(*args, torch.float32).numpy(),
            "unrounded64": unrounded(*args, torch.float64).numpy(),
            "fp64_bf16": direct_bf16(unrounded(*args, torch.float64)).numpy(),
            "direct_bf16_pv": par.direct_bf16_pv(*args, heads, kv_heads, d, scale).numpy(),
        }
        for tile in (2, 5, 16, 512):
            rec[f"tiled_{tile}"] = par.tiled_bf16_pv(*args, heads, kv_heads, d, scale, tile).numpy()
        for key, value in rec.items():
            out[f"{name}/{key}"] = np.asarray(value)
    out["names"] = np.array([c[0] for c in cases])
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **out)


def softcap_window_cases(ref_tests):
    fn = lift(os.path.join(ref_tests, "paged_attention_generalized_smoke.py"), "cpu_ref_attention",
              {"torch": torch})
    gen = torch.Generator().manual_seed(20261102)
    out, names = {}, []
    for name, heads, kv_heads, d, seqs, softcap, window in (
            ("softcap_swa", 4, 2, 64, [(0, 20), (11, 1)], 50.0, 8),
            ("swa_only", 6, 3, 64, [(5, 3), (30, 1)], 0.0, 16),
            ("softcap_only", 2, 1, 128, [(0, 9)], 30.0, -1)):
        slots = 128
        kp = torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16)
        vp = torch.randn(slots, kv_heads, d, generator=gen).to(torch.bfloat16)
        context = max(p + l for p, l in seqs)
        mapping = torch.zeros(len(seqs), context, dtype=torch.int32)
        metas, cursor, row = [], 1, 0
        for i, (prefix, length) in enumerate(seqs):
            ids = list(range(cursor, cursor + prefix + length))
            cursor += prefix + length + 2
            mapping[i, : prefix + length] = torch.tensor(ids, dtype=torch.int32)
            metas.append((row, prefix, length, ids))
            row += length
        q = torch.randn(row, heads, d, generator=gen).to(torch.bfloat16)
        scale = 1.0 / math.sqrt(d)
        ref = fn(q, kp, vp, metas, scale, softcap, window)
        requests = np.array([i for i, (_, l) in enumerate(seqs) for _ in range(l)], dtype=np.int64)
        positions = np.array([p + j for p, l in seqs for j in range(l)], dtype=np.int64)
        rec = {"heads": heads, "kv_heads": kv_heads, "head_dim": d, "scale": np.float64(scale),
               "softcap": np.float64(softcap), "window": window, "mapping": mapping.numpy(),
               "requests": requests, "positions": positions, "q": bits(q.reshape(row, heads * d)),
               "key_pool": bits(kp), "value_pool": bits(vp), "out_bf16": bits(ref.reshape(row, heads * d))}
        for key, value in rec.items():
            out[f"{name}/{key}"] = np.asarray(value)
        names.append(name)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "softcap_window.npz"), **out)


def rounding_cases():
    from fp64_reference import direct_bf16
    from decoder_cpu_reference import store_boundary
    gen = torch.Generator().manual_seed(20261103)
    x = torch.randn(4096, generator=gen, dtype=torch.float64) * torch.logspace(-42, 38, 4096, dtype=torch.float64)
    edge = torch.tensor([0.0, -0.0, 1.0, 1 + 2**-8, 1 + 2**-8 + 2**-32, 1 + 2**-8 - 2**-40, 1 + 3 * 2**-8,
                         2.0**-126, 2.0**-127, 2.0**-133, 2.0**-134, 1.5 * 2.0**-134, 2.0**-135,
                         3.3895313892515355e38, 3.4e38, -3.4e38, 65504.0, 1e-40, -1e-40], dtype=torch.float64)
    values = torch.cat((x, edge))
    np.savez_compressed(os.path.join(HERE, "rounding.npz"), x=values.numpy(),
                        direct_bf16=direct_bf16(values).numpy(),
                        store_boundary64=store_boundary(values).numpy(),
                        store_boundary32=store_boundary(values.float()).numpy())


def norm_rotary_cases(ref_tests):
    from fp64_reference import direct_bf16
    eps = 1e-6
    env = {"torch": torch, "direct_bf16": direct_bf16, "EPSILON": eps,
           "EPSILON_FP32": torch.tensor(eps, dtype=torch.float32).item()}
    norm_ref = lift(os.path.join(ref_tests, "fused_add_rms_fx_smoke.py"), "reference", env)
    rot_ref = lift(os.path.join(ref_tests, "rotary_runtime_smoke.py"), "reference",
                   {"torch": torch, "direct_bf16": direct_bf16})
    gen = torch.Generator().manual_seed(20261104)
    out = {"epsilon": np.float64(eps)}
    x = torch.randn(5, 192, generator=gen).to(torch.bfloat16)
    res = torch.randn(5, 192, generator=gen).to(torch.bfloat16)
    gamma = (torch.randn(192, generator=gen) * 0.1 + 1).to(torch.bfloat16)
    out.update(norm_x=bits(x), norm_res=bits(res), norm_gamma=bits(gamma))
    for fp64 in (False, True):
        y, u = norm_ref(x, res, gamma, None, fp64)
        out[f"norm_y_{'64' if fp64 else '32'}"] = y.numpy()
        out[f"norm_u_{'64' if fp64 else '32'}"] = u.numpy()
    for tag, heads, head_dim, rotary_dim in (("full", 3, 64, 64), ("partial", 2, 96, 62)):
        cache = torch.randn(40, rotary_dim, generator=gen).to(torch.bfloat16)
        xin = torch.randn(6, heads * head_dim, generator=gen).to(torch.bfloat16)
        pos = torch.randint(0, 40, (6,), generator=gen)
        out.update({f"rot_{tag}_x": bits(xin), f"rot_{tag}_cache": bits(cache), f"rot_{tag}_pos": pos.numpy(),
                    f"rot_{tag}_geom": np.array([heads, head_dim, rotary_dim])})
        for neox in (True, False):
            for fp64 in (False, True):
                key = f"rot_{tag}_{'neox' if neox else 'gptj'}_{'64' if fp64 else '32'}"
                out[key] = rot_ref(xin, cache, pos, head_dim, rotary_dim, neox, fp64).numpy()
    np.savez_compressed(os.path.join(HERE, "norm_rotary.npz"), **out)


def after_attention_cases(ref_tests):
    """Grammar bitmask and rank-ordered sum: the reference's own CPU functions, lifted from its device tests
    (``tests/vocab_bitmask_device_smoke.py``, ``tests/tp4_gather_reduce_smoke.py``)."""
    env = {"torch": torch}
    ref_mask = lift(os.path.join(ref_tests, "vocab_bitmask_device_smoke.py"), "ref_apply_bitmask", env)
    rank_sum = lift(os.path.join(ref_tests, "tp4_gather_reduce_smoke.py"), "_canonical_rank_sum", env)
    gen = torch.Generator().manual_seed(20261177)
    out = {}
    cases = [("bf16_35", torch.bfloat16, 1, 35, None, -1, False), ("bf16_1025", torch.bfloat16, 3, 1025, None, -1, False),
             ("f32_1025_tail", torch.float32, 3, 1025, None, -1, True), ("f32_40_short", torch.float32, 2, 40, None, -1, True),
             ("bf16_40_short", torch.bfloat16, 2, 40, None, -1, False), ("f32_rows", torch.float32, 4, 64, [2, 0, 2], -1, False),
             ("bf16_vocab", torch.bfloat16, 3, 200, None, 150, True)]
    for name, dtype, batch, vocab, indices, vocab_size, mask_tail in cases:
        words = 1 if name.endswith("short") else (vocab + 31) // 32
        logits = (torch.randn(batch, vocab, generator=gen) * 3).to(dtype)
        mask = torch.randint(-2 ** 31, 2 ** 31 - 1, (batch, words), generator=gen, dtype=torch.int64).to(torch.int32)
        idx = None if indices is None else torch.tensor(indices, dtype=torch.int32)
        want = ref_mask(logits, mask, idx, vocab_size, mask_tail)
        raw = (lambda t: bits(t)) if dtype == torch.bfloat16 else (lambda t: t.numpy().view(np.uint32).copy())
        out[f"mask_{name}_logits"], out[f"mask_{name}_mask"], out[f"mask_{name}_out"] = raw(logits), mask.numpy(), raw(want)
        out[f"mask_{name}_args"] = np.array([vocab_size, int(mask_tail)] + ([] if indices is None else indices), dtype=np.int64)
    for world in (1, 2, 4, 8):
        parts = [(torch.randn(1536, generator=gen) * 10 ** float(torch.randn((), generator=gen))).to(torch.bfloat16)
                 for _ in range(world)]
        out[f"sum_{world}_parts"] = np.stack([bits(t) for t in parts])
        out[f"sum_{world}_out"] = bits(rank_sum(parts))
    np.savez_compressed(os.path.join(HERE, "after_attention.npz"), **out)


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    ref = sys.argv[1]
    ref_tests = os.path.join(ref, "tests")
    sys.path.insert(0, ref_tests)
    torch.set_num_threads(2)
    attention_cases(ref_tests)
    softcap_window_cases(ref_tests)
    rounding_cases()
    norm_rotary_cases(ref_tests)
    after_attention_cases(ref_tests)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
