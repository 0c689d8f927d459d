"""Generates tests/golden/ref_*.npz by running the reference's own CUDA kernels (compiled
unmodified into oracle/_ref by oracle/Makefile) on a GPU.  Run on a machine with a CUDA device:

    python tests/golden/make_golden.py [output_dir]

Each file holds seeded inputs and the outputs of the reference's eleven-kernel batch-norm +
ReLU layer (oracle/ref_gpu.py gives the order and the reference line numbers).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_gpu  # noqa: E402

CASES = [  # name, shape, seed, loc, scale, block_sz
    ("tiny2d", (4, 3, 5, 5), 11, 0.0, 1.0, 1024),
    ("odd2d", (5, 3, 7, 7), 12, 0.5, 2.0, 256),
    ("mid2d", (16, 3, 14, 14), 13, 0.5, 2.0, 1024),
    ("vol3d", (2, 4, 3, 6, 8), 14, 0.0, 1.0, 512),
]


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out, exist_ok=True)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for name, shape, seed, loc, scale, block in CASES:
        rng = np.random.default_rng(seed)
        x = (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale) + np.float32(loc))
        dy = rng.standard_normal(shape, dtype=np.float32)
        c = shape[1]
        rm0, rv0 = np.zeros(c, np.float32), np.ones(c, np.float32)
        cfg = ref_gpu.KernelConfig(block, 32 * sms)
        r = ref_gpu.bn_relu_fwd_bwd(torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda(), 1e-5, 0.1,
                                    torch.from_numpy(rm0).cuda(), torch.from_numpy(rv0).cuda(), cfg=cfg)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out, "ref_%s.npz" % name), x=x, dy=dy, eps=np.float32(1e-5),
                            avg_rate=np.float32(0.1), block_sz=np.int32(block), run_mean0=rm0, run_var0=rv0,
                            **{k: v.cpu().numpy() for k, v in r.items()})
        print("wrote", name, shape)


if __name__ == "__main__":
    main()
