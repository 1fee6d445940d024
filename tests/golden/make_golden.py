"""Regenerate tests/golden/*.npz and evictor_*.json from the REFERENCE ITSELF.

Runs the scenarios of tests/scenarios.py and the eviction-policy sequences of
tests/evictor_cases.py against oracle/_ref/libtorpor_ref_fake.so -- the reference's
own headers (include/server/{memory_manager,block_manager,model_repo,evictor,controller}.hpp)
compiled where they lie against a host-memory CUDA stand-in -- and stores the
recorded tables, victims, scheduling decisions and controller traces.  Needs the reference tree to build that library:

    make -C oracle ref && python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import scenarios  # noqa: E402
import evictor_cases  # noqa: E402
import scheduler_cases  # noqa: E402
import controller_cases  # noqa: E402


def main():
    backend = scenarios.TsoBackend("ref_fake")
    for name in scenarios.SCENARIOS:
        rec = scenarios.run(backend, name)
        np.savez_compressed(scenarios.golden_path(name), **rec)
        print(name, len(rec), "records,", os.path.getsize(scenarios.golden_path(name)), "bytes")
    for kind in ("LRU", "IA"):
        cases = evictor_cases.record(backend.lib, kind)
        path = os.path.join(HERE, f"evictor_{kind}.json")
        with open(path, "w") as f:
            json.dump(cases, f)
        print("evictor", kind, len(cases), "sequences,", os.path.getsize(path), "bytes")
    # the reference's Controller object itself (controller.hpp compiled where it lies)
    for policy in ("IA", "RAND"):
        runs = scheduler_cases.record(backend, policy)
        path = os.path.join(HERE, f"scheduler_{policy}.json")
        with open(path, "w") as f:
            json.dump(runs, f)
        print("scheduler", policy, len(runs), "streams,", sum(len(r) for r in runs), "decisions,", os.path.getsize(path), "bytes")
    # ... and its own loop (Controller::start), one scripted event at a time
    for sp, ep in controller_cases.COMBOS:
        runs = controller_cases.record(backend, sp, ep)
        path = os.path.join(HERE, f"controller_{sp}_{ep}.json")
        with open(path, "w") as f:
            json.dump(runs, f, separators=(",", ":"))
        print("controller", sp, ep, len(runs), "streams,", sum(len(r) for r in runs), "events,", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
