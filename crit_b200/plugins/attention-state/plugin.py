"""crit plugin shell for the kv_cache slot (same id, options and entry points as crit's attention-state plugin:
inference/attention-state/plugin.py:132-151), backed by crit_b200's pool and kernels."""
from crit_b200.kv_state import KVStateCache


def _device(context):
    """The device the engine runs on: the load context's, or CUDA when torch has it (a plugin's own tests)."""
    device = getattr(context, "device", None)
    if device is None:
        import torch
        device = "cuda" if torch.cuda.is_available() else "cpu"
    return str(device)


def _on_cuda(context):
    return _device(context).startswith("cuda")


def memory(context, options):
    """The fresh buffer the plugin makes on a CUDA engine (fresh_mib), exactly; pools allocate when the model makes
    them (inference/attention-state/plugin.py:132-137)."""
    return {"device": (int(options.get("fresh_mib") or 0) << 20) if _on_cuda(context) else 0, "host": 0}


def create(context, options, parts):
    if options.get("kernels", "auto") != "auto":
        raise ValueError("crit_b200's attention-state writes pages with its CUDA kernels only (kernels: auto)")
    if options.get("elastic") or options.get("host_pages_mib"):
        raise ValueError("crit_b200's attention-state does not serve elastic pages")
    import crit_b200
    fresh = None
    if _on_cuda(context) and options.get("fresh_mib"):
        import torch
        from crit_b200.pool import FreshBuffer
        fresh = FreshBuffer(torch.empty(int(options["fresh_mib"]) << 20, dtype=torch.uint8, device=_device(context)))
    return KVStateCache(options["page"], options["step_rows"], options["step_tokens"], options["window"],
                        options["round_rows"], crit_b200, fresh=fresh)
