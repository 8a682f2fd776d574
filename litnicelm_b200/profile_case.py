"""Small fixed case for profilers: a few forwards of one benchmark shape.

    python -m litnicelm_b200.profile_case --workload c2 --context 640 --repeats 4

Builds seeded synthetic weights, runs `repeats` whole-context forwards (the work
of one generated token) at the given context length through the C ABI and
prints the device time of each. Kept short so that a profiler capture ends by
itself.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import formats
from .plugin import Session


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2", choices=sorted(formats.CONFIG_DIMS))
    ap.add_argument("--context", type=int, default=640)
    ap.add_argument("--streams", type=int, default=1)
    ap.add_argument("--repeats", type=int, default=4)
    ap.add_argument("--generate", type=int, default=0, help="also decode this many tokens")
    args = ap.parse_args()
    d = formats.CONFIG_DIMS[args.workload]
    arena = formats.make_param_arena(d, 1002)
    ids = np.stack([formats.zipf_prompt(d.vocab, args.context, 4000 + i) for i in range(args.streams)])
    times = []
    with Session(d, args.streams) as s:
        s.load_params(arena)
        for _ in range(args.repeats):
            s.forward(ids)
            st = s.stats()
            times.append(st.device_ms)
        out = {"workload": args.workload, "context": args.context, "streams": args.streams,
               "forward_ms": times, "kernel_launches_per_forward": int(st.kernel_launches)}
        if args.generate:
            s.generate(ids, args.generate)
            st = s.stats()
            out["generate_ms"] = st.device_ms
            out["generate_tokens"] = int(st.tokens)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
