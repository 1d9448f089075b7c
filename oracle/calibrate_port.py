"""Calibration of the CPU port against the reference's own PyTorch modules (test infrastructure).

bench.py's CPU legs time the numpy port in oracle/pikv_oracle.py because the reference's modules cannot
travel to the GPU box.  This script runs BOTH, on the same host and the same config-2 inputs, where the
reference is available, and prints one JSON line with the two times and their ratio:

  reference  gate tail       = the Linear producing the logits + softmax + top-k + renormalisation
                               (core/single/pikv_routing.py:65-79)
             quantise        = module QuantizedCompressor.forward on K and V, int8 symmetric, group 128
                               (core/single/module/pikv_compression.py:1014-1051)
  port       bench.cpu_step  = the same gate tail + slot scan + per-(token, head) quantisation + scatter

    python oracle/calibrate_port.py --reference /path/to/PiKV [--threads N]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--repeats", type=int, default=5)
    a = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, ROOT)
    sys.path.insert(0, a.reference)
    import bench
    nthreads = a.threads or bench.host_threads()
    import torch
    torch.set_num_threads(nthreads)
    from core.single.module import pikv_compression as ref_c

    cfg = bench.WORKLOAD
    T, H, E, k = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["top_k"]
    kv = cfg["kv_heads"] * cfg["head_dim"]
    act, K, V = bench.synth_inputs(T, H, E, kv, 1)
    w2, b2 = bench.gate_weights(H, E, 7)
    actf, Kf, Vf = act.float(), K.float()[None], V.float()[None]
    lin = torch.nn.Linear(H, E)
    lin.weight.data.copy_(w2.float())
    lin.bias.data.copy_(b2)
    qc = ref_c.QuantizedCompressor(kv, bits=8, group_size=128, symmetric=True).eval()

    def ref_step():
        with torch.no_grad():
            logits = lin(actf)                                     # pikv_routing.py:66 (last layer of the gate net)
            probs = torch.softmax(logits, dim=-1)                  # :73
            top_p, top_i = torch.topk(probs, k, dim=-1)            # :76
            top_p = top_p / top_p.sum(dim=-1, keepdim=True)        # :79
            return qc(Kf, Vf), top_i

    def med(fn, n):
        fn()
        ts = []
        for _ in range(n):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return sorted(ts)[len(ts) // 2]

    t_ref = med(ref_step, a.repeats)
    _, dt_port, _ = bench.run_cpu(a.repeats, 1, T)
    print(json.dumps({"tokens": T, "threads": nthreads, "reference_s": t_ref, "port_s": dt_port,
                      "port_over_reference": dt_port / t_ref,
                      "reference_tokens_per_s": T / t_ref, "port_tokens_per_s": T / dt_port}))


if __name__ == "__main__":
    main()
