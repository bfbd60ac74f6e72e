"""Runs a script of this repository with the device entry points replaced by their host model (tests/cpu_kernel_model.py):

    python tests/run_with_kernel_model.py <script.py> [its arguments]

Under torchrun (WORLD_SIZE > 1) the ranks are taken to be real processes that share the heap, so barriers and waits are
real; FL_MODEL_LOCK names the file that stands in for system-scope atomics.  The tests use it to run experiment scripts
end to end on a machine without a GPU (the scripts are started with their own ``--device cpu``)."""
import os
import runpy
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import cpu_kernel_model

if __name__ == "__main__":
    script = sys.argv[1]
    sys.argv = sys.argv[1:]
    multi = int(os.environ.get("WORLD_SIZE", "1")) > 1
    with cpu_kernel_model.installed(single_process=not multi, lock_path=os.environ.get("FL_MODEL_LOCK")) as model:
        model.wait_limit_s = float(os.environ.get("FL_MODEL_WAIT_S", "60"))
        runpy.run_path(script, run_name="__main__")
