"""crit plugin shell for the kv_cache slot (same id, options and entry points as crit's attention-state plugin:
inference/attention-state/plugin.py:132-151), backed by crit_b200's pool and kernels."""
from crit_b200.kv_state import KVStateCache


def memory(context, options):
    """Nothing is allocated when the plugin is made: pools allocate when the model makes them."""
    return {"device": 0, "host": 0}


def create(context, options, parts):
    if options.get("kernels", "auto") != "auto":
        raise ValueError("crit_b200's attention-state writes pages with its CUDA kernels only (kernels: auto)")
    if options.get("fresh_mib") or options.get("elastic") or options.get("host_pages_mib"):
        raise ValueError("crit_b200's attention-state does not serve fresh buffers or elastic pages")
    import crit_b200
    return KVStateCache(options["page"], options["step_rows"], options["step_tokens"], options["window"],
                        options["round_rows"], crit_b200)
