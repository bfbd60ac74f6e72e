"""fuselink_b200 — a Blackwell-native multi-path GPU communication framework.

Layers (bottom up):

* ``csrc/``      sm_100a kernels (tcgen05 grouped GEMM, fused dispatch/combine, embedding-bag + all-to-all,
                 KV pack + transfer, chunked peer copies), the cuMem region layer, the idleness monitor and
                 the ncclNet plugin (``lib/libnccl-net-fuselink.so``).
* ``parallel/``  symmetric heap over cuMem regions, path selector, process-group helpers.
* ``ops/``       Python entry points of the kernels plus plain-PyTorch fp32 references.
* ``models/``    MoE expert-parallel layer, DLRM, Llama-shaped prefill/decode used by the serving path.
* ``serving/``   disaggregated prefill -> decode pipeline and trace replay.
* ``utils/``     env knobs, timing, clocks sampling, roofline arithmetic.
"""
from ._ext import C, have_native, require_native  # noqa: F401

__version__ = "0.1.0"


def stats(selector=None) -> dict:
    """Observability snapshot: cuMem bytes held per device and, when a selector is given, per-path state."""
    out = {"native": have_native()}
    if have_native():
        out["vmm_backend"] = C.vmm_backend()
        out["vmm_bytes"] = {d: C.vmm_usage(d) for d in range(8) if C.vmm_usage(d)}
    if selector is not None:
        out["paths"] = [vars(s) for s in selector.stats()]
        out["selector"] = {"direct": selector.direct_answers, "relay": selector.relay_answers}
    return out
