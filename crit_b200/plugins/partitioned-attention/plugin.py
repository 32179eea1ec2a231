"""crit plugin shell for the attention slot (same id, options and entry points as crit's partitioned-attention plugin:
inference/partitioned-attention/plugin.py:67-103), backed by crit_b200's attention and kernels."""
from crit_b200.attention import DeviceAttention, PartitionedAttention


def memory(context, options):
    """The split-K partials come from the engine's scratch (workspace_mib at most) or the kernels' own workspace:
    nothing is allocated when the plugin is made."""
    return {"device": 0, "host": 0}


def create(context, options, parts):
    if options.get("kernels", "auto") != "auto" or options.get("flashinfer", "off") != "off":
        raise ValueError("crit_b200's partitioned-attention reads pages with its CUDA kernels only (kernels auto, flashinfer off)")
    reader = options.get("prompt_reader", "auto")
    form = DeviceAttention(None, "auto", partitions=options.get("partitions", 0), piece=options.get("piece", 0),
                           device=getattr(context, "device", None), kernels_mib=options.get("workspace_mib", 128),
                           prompt_reader="prefill" if reader == "auto" else reader,
                           scratch=getattr(context, "scratch", None),
                           window_engine=options.get("window_engine", "auto"))
    return PartitionedAttention(parts["kv_cache"], options, form)
