"""B200-native MegaMoE expert backend behind the operator surface of the ``vllm_sm107_megamoe`` plugin.

``register()`` is the vLLM general-plugin entry point (``vllm_sm107_megamoe/__init__.py:9-31`` of the reference): a
no-op unless the plugin is named in ``VLLM_PLUGINS``, otherwise it registers the out-of-tree ``DeepGemmMegaMoEExperts``
layer class.  Importing this package imports neither torch, vLLM nor the CUDA library.
"""

import os

PLUGIN_NAME = "b200_megamoe"


def register() -> None:
    allowed = os.environ.get("VLLM_PLUGINS")
    if allowed is None or PLUGIN_NAME not in [p.strip() for p in allowed.split(",")]:
        return
    from vllm.model_executor.custom_op import PluggableLayer
    try:
        from vllm.model_executor.layers.fused_moe.deep_gemm_mega_moe import DeepGemmMegaMoEExperts
    except ImportError as exc:
        raise RuntimeError("This vLLM has no DeepGemmMegaMoEExperts layer; apply the MegaMoE plugin hook") from exc
    if not issubclass(DeepGemmMegaMoEExperts, PluggableLayer) or not hasattr(DeepGemmMegaMoEExperts, "_import_backend"):
        raise RuntimeError("DeepGemmMegaMoEExperts lacks the PluggableLayer hook (`_import_backend`)")
    from .experts import make_experts_class

    PluggableLayer.register_oot(make_experts_class(DeepGemmMegaMoEExperts), name="DeepGemmMegaMoEExperts")
