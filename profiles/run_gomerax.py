"""One prompt portion of 2048 tokens and a few decode steps of a three-layer Gomerax model (width 2048: windowed latent attention with a rotated
part and a sink; a dense feed-forward, then routed experts in groups with a shared expert; layers 1 and 2 run twice) through the engine's own
step: the workload of the launch lists and ncu captures of the Gomerax kernels.  python profiles/run_gomerax.py [decode steps]"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aha_b200 import B200Model, synth     # noqa: E402

steps = int(sys.argv[1]) if len(sys.argv) > 1 else 3
cfg = synth.gomerax_shape(width=2048, n_layers=3, heads=16, head_dim=128, rot_dim=64, ff=8192, experts=16, top=2, expert_ff=2048, vocab=8000, kv_rank=512, q_rank=1024, window=1024,
                          max_positions=4096, loop=(1, 3, 2))
m = B200Model("gomerax", cfg, synth.make_gomerax(cfg, 0, fast=True), max_ctx=4096, max_prefill=2048, max_seqs=2, use_graph=False)
ids = np.random.default_rng(0).integers(0, 8000, 2048 + steps).astype(np.uint32)
s = m.seq_open()
m.feed([(s, ids[:2048], [2047])])
for t in range(steps):
    m.feed([(s, ids[2048 + t:2049 + t], [0])])
m.seq_close(s)
print("kernel launches", m.stats()["kernel_launches"])
m.close()
