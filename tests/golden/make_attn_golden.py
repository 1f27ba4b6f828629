"""Generates tests/golden/attn_simple_*.npz by EXECUTING the reference's own
attention math: the function bodies of ``make_rand`` and ``simple_attn`` are
taken from the reference's torch_attn.py at run time (the file cannot be
imported whole because it loads a shared library at top level), executed on
torch CPU, and their inputs/outputs stored.  Nothing of the reference is copied
into this repository; only the numbers are.

    python tests/golden/make_attn_golden.py /path/to/reference

Inputs are rounded to fp16 first (the kernels under test take fp16), the
reference math then runs in fp32 on those values.
"""
import ast
import math
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_attn_golden.py /path/to/reference")
REF = sys.argv[1]
HERE = os.path.dirname(os.path.abspath(__file__))


def reference_functions():
    src = open(os.path.join(REF, "torch_attn.py")).read()
    tree = ast.parse(src)
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in ("make_rand", "simple_attn")]
    assert len(wanted) == 2
    ns = {"math": math, "torch": torch}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), "torch_attn.py", "exec"), ns)
    return ns["make_rand"], ns["simple_attn"]


def main():
    make_rand, simple_attn = reference_functions()
    # (N, d, seeds): the reference's testbed size (attn_main.hpp:2-3), its script's
    # seeds (torch_attn.py:27-29), and a head_dim-128 case shaped like the headline config.
    for name, N, d, seeds, signed in (("n256_d64", 256, 64, (101, 237, 280), False),
                                      ("n320_d128", 320, 128, (101, 237, 280), True)):
        q, k, v = (make_rand(N, d, s) for s in seeds)
        if signed:
            # the reference's generator is non-negative; centre it so that softmax sees both signs
            q, k, v = (4.0 * (t - t.mean()) for t in (q, k, v))
        q16, k16, v16 = (t.to(torch.float16) for t in (q, k, v))
        o = simple_attn(q16.float(), k16.float(), v16.float())
        o_scale1 = simple_attn(q16.float(), k16.float(), v16.float(), scale=1)
        np.savez_compressed(os.path.join(HERE, f"attn_simple_{name}.npz"),
                            q=q16.numpy(), k=k16.numpy(), v=v16.numpy(),
                            o=o.numpy().astype(np.float32), o_scale1=o_scale1.numpy().astype(np.float32))
        print(name, "written", o.shape, float(o.abs().max()))
    # the reference interface's own element type and testbed size (attn_main.hpp:2-3): bfloat16, N=256, d=64
    q, k, v = (make_rand(256, 64, s) for s in (101, 237, 280))
    qb, kb, vb = (t.to(torch.bfloat16) for t in (q, k, v))
    o = simple_attn(qb.float(), kb.float(), vb.float())
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "attn_simple_n256_d64_bf16.npz"), q_bits=bits(qb), k_bits=bits(kb),
                        v_bits=bits(vb), o=o.numpy().astype(np.float32))
    print("n256_d64_bf16 written", o.shape)


if __name__ == "__main__":
    main()
