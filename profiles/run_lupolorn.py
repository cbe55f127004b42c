"""One prompt portion of 2048 tokens and a few decode steps of a four-layer Lupolorn model (width 2048: attention, minGRU, latent attention,
attention; dense and routed feed-forwards in turn) through the engine's own step: the workload of the launch lists and ncu captures of
the Lupolorn kernels.  python profiles/run_lupolorn.py [decode steps]"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aha_b200 import B200Model, synth     # noqa: E402

steps = int(sys.argv[1]) if len(sys.argv) > 1 else 3
cfg = synth.lupolorn_shape(width=2048, n_layers=4, heads=16, kv_heads=4, head_dim=128, ff=8192, experts=16, top=2, expert_ff=2048, vocab=8000, kv_rank=512, q_rank=1024, window=1024)
m = B200Model("lupolorn", cfg, synth.make_lupolorn(cfg, 0, fast=True), max_ctx=4096, max_prefill=2048, max_seqs=2)
ids = np.random.default_rng(0).integers(0, 8000, 2048 + steps).astype(np.uint32)
s = m.seq_open()
m.feed([(s, ids[:2048], [2047])])
for t in range(steps):
    m.feed([(s, ids[2048 + t:2049 + t], [0])])
m.seq_close(s)
print("kernel launches", m.stats()["kernel_launches"])
m.close()
