"""Generate kernel-level golden fixtures by RUNNING the reference's compiled CUDA kernel on a GPU.

    python oracle/build_ref.py            # where the reference checkout is available
    python tests/golden/make_golden_gpu.py [outdir]      # on a machine with a GPU

Loads ``oracle/_ref/FastAttention2/kernel.so`` (the reference's ``combined_kernel_general.cu``
compiled unmodified) and records, for a handful of small shapes, the outputs of
``kernel.<dtype>(Q, K, V, 1, False, reversed)`` and of the three permuted calls of
``CustomAttention.backward`` (``Cuda_Kernel/Custom_Kernel.py:106-108``).  The ``.npz`` files it
writes are committed next to this script.  Nothing here is imported by the product.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from conftest import load_reference_kernel  # noqa: E402

# (name, dtype, B, H, S, Dk, Dv)
CASES = [
    ("f64_gradcheck_shape", torch.float64, 1, 2, 63, 128, 128),   # Custom_Kernel.py:157
    ("f32_d64", torch.float32, 2, 2, 100, 64, 64),
    ("f32_d32_halfwarp", torch.float32, 1, 2, 70, 32, 32),         # combined_kernel_general.cu:273-277
    ("f32_dv_ne_dk", torch.float32, 1, 2, 65, 64, 32),             # speeds.py:4-6,137
    ("bf16_d64", torch.bfloat16, 1, 2, 96, 64, 64),
    ("f16_d128", torch.float16, 1, 1, 80, 128, 128),
]


def main(outdir):
    ref = load_reference_kernel()
    assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    os.makedirs(outdir, exist_ok=True)
    fn = {torch.float64: ref.float64, torch.float32: ref.float32, torch.bfloat16: ref.bfloat16,
          torch.float16: ref.float16}
    for name, dt, B, H, S, Dk, Dv in CASES:
        g = torch.Generator().manual_seed(sum(map(ord, name)))
        q = torch.randn(B, H, S, Dk, generator=g)
        k = torch.randn(B, H, S, Dk, generator=g)
        v = torch.randn(B, H, S, Dv, generator=g)
        do = torch.randn(B, H, S, Dv, generator=g)
        q = torch.nn.functional.normalize(q, dim=-1)
        k = torch.nn.functional.normalize(k, dim=-1)
        # values exactly representable in the case's dtype, stored as float32
        q, k, v, do = (t.to(dt).float() if dt != torch.float64 else t for t in (q, k, v, do))
        Q, K, V, DO = (t.to(dt).cuda() for t in (q, k, v, do))
        f = fn[dt]
        out = f(Q, K, V, 1, False, False)
        out_rev = f(Q, K, V, 1, False, True)
        rec = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), dout=do.numpy(),
                   out=out.double().cpu().numpy(), out_rev=out_rev.double().cpu().numpy())
        if Dv % 16 == 0 and Dv >= 32:
            rec["dq"] = f(DO, V, K, 1, False, False).double().cpu().numpy()
            rec["dk"] = f(V, DO, Q, 1, False, True).double().cpu().numpy()
            rec["dv"] = f(K, Q, DO, 1, False, True).double().cpu().numpy()
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(outdir, f"kernel_ref_{name}.npz"), **rec)
        print(name, "ok", float(np.abs(rec["out"]).max()))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
