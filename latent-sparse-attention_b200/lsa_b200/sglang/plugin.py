"""The plugin entry point: one standing hook on the model config, the design's hooks once a config names a design.

The reference registers itself as `[project.entry-points."sglang.srt.plugins"] lsa = "lsa.sglang.plugin:register"`
(`pyproject.toml:147-148`) and this module keeps that contract (`src/lsa/sglang/plugin.py:228-250,339-354,858-1010`):

  register()    called once a process by sglang's plugin loader: puts one AFTER hook on `ModelConfig.__init__`.
  configure()   that hook: finds the `"lsa"` block of the model config and enables the design it names.
  enable_lsa()  resolves EVERY target before registering ANY hook, so an upstream rename fails with the name in the
                message instead of leaving a server that runs the checkpoint's own attention under an LSA label.

SGLang's `HookRegistry` is imported at call time only; tests pass a registry of their own.
"""

from __future__ import annotations

import importlib
import logging
from typing import Any

from lsa_b200.sglang import backend, settings
from lsa_b200.sglang.settings import DesignSettings

logger = logging.getLogger(__name__)

BANNER_READY = "lsa: enabled"  # what a launcher greps a server's log for (src/lsa/sglang/constants.py:9-24)

# Where a server's settings arrive, and so the one hook every server carries
MODEL_CONFIG = "sglang.srt.configs.model_config.ModelConfig.__init__"

# The grouped-query attention backends a design patches, and the methods of each
GROUPED_QUERY_BACKENDS = (
    "sglang.srt.layers.attention.flashattention_backend.FlashAttentionBackend",
    "sglang.srt.layers.attention.triton_backend.TritonAttnBackend",
)
GROUPED_QUERY_METHODS = ("__init__", "init_forward_metadata", "init_forward_metadata_out_graph", "forward_extend",
                         "forward_decode")
GROUPED_QUERY_TARGETS = tuple(f"{attention}.{method}" for attention in GROUPED_QUERY_BACKENDS
                              for method in GROUPED_QUERY_METHODS)
HOOK_REGISTRY = "sglang.srt.plugins.hook_registry"
# Where a decode runner captures its graphs, and the getter that says which attention variant is being captured: both
# must be there for a graph a context range (plugin.py:138-143); a runner without them keeps its one decode graph
CONTEXT_GRAPH_TARGETS = (
    "sglang.srt.model_executor.runner.decode_cuda_graph_runner.DecodeCudaGraphRunner._capture_one_stream",
    "sglang.srt.model_executor.runner_utils.capture_mode.get_capture_attention_variant",
)

# The design a process serves, once a model config named one
ENABLED: dict = {}


def resolve(target: str) -> object:
    """The object a dotted `module.attr` or `module.Class.method` path names (plugin.py:228-248)."""
    module_path, _, attribute = target.rpartition(".")
    try:
        holder: Any = importlib.import_module(module_path)
    except ModuleNotFoundError:
        outer, _, class_name = module_path.rpartition(".")
        holder = getattr(importlib.import_module(outer), class_name)
    return getattr(holder, attribute)


def unresolved(targets: tuple) -> list:
    """The targets that no longer resolve, each with why (plugin.py:339-354)."""
    missing = []
    for target in targets:
        try:
            resolve(target)
        except (AttributeError, ModuleNotFoundError, ImportError, ValueError) as failure:
            missing.append(f"{target} ({failure})")
    return missing


def _registry(registry=None):
    if registry is not None:
        return registry, registry.HookType
    module = importlib.import_module(HOOK_REGISTRY)
    return module.HookRegistry, module.HookType


def enable(result: None, self: Any, *args: Any, **kwargs: Any) -> None:
    """AFTER hook of an attention backend's `__init__`: give the backend an indexer for every quadratic layer of a
    grouped-query model, built from the design the model config named (`models/qwen3_5/backend.py:305-347`).

    Raises:
        TypeError: The backend was built without a model runner.
    """
    runner = kwargs.get("model_runner", args[0] if args else None)
    if runner is None:
        raise TypeError("the attention backend was built without a model runner")
    if not hasattr(self, "lsa_indexers"):
        self.lsa_indexers = {}
    design = ENABLED.get("design")
    if design is not None:
        backend.enable(self, runner, design)


def maintain(*args: Any, **kwargs: Any) -> None:
    """BEFORE hook of `init_forward_metadata` and of `init_forward_metadata_out_graph`: the index's host-side upkeep
    of a step - the clustering of blocks that closed, page allocation - runs here, before the forward and outside
    any captured graph (plugin.py:491-522)."""
    backend_object = args[0] if args else kwargs.get("self")
    forward_batch = kwargs.get("forward_batch", args[1] if len(args) > 1 else None)
    in_capture = kwargs.get("in_capture", args[2] if len(args) > 2 else False)
    if forward_batch is None or in_capture or not getattr(backend_object, "lsa_indexers", None):
        return
    backend.maintain_all(backend_object, forward_batch)


def capture_context_graphs(original: Any, self: Any, *args: Any, **kwargs: Any) -> Any:
    """AROUND hook of the decode runner's graph capture: hand it one graph a context range of the design, unless the
    runner already captures variants of its own or the step is not a flat decode (plugin.py:600-631). What a graph
    computes is the same; a range trims the page-table columns no request of it can fill."""
    from lsa_b200.sglang import context_buckets

    design = ENABLED.get("design")
    flat_decode = design is not None and design.serving.decode == "flat" and self.capture_forward_mode.is_decode()
    if flat_decode and getattr(self, "attention_graph_variants", None) is None:
        longest = self.model_runner.model_config.context_len
        ranges = context_buckets.ContextBuckets.under(design.serving.decode_context_limits, longest)
        if ranges is not None:
            logger.info("lsa: decode graphs for contexts up to %s and %d", ranges.limits, longest)
            self.attention_graph_variants = ranges
    return original(self, *args, **kwargs)


def context_graphs(hook_registry, kinds, targets: tuple = CONTEXT_GRAPH_TARGETS) -> bool:
    """Register the capture hook where this sglang keys decode graphs by an attention variant; elsewhere the server
    keeps one decode graph, which serves every context (plugin.py:680-702)."""
    missing = unresolved(targets)
    if missing:
        logger.info("lsa: one decode graph, no context ranges - %s", "; ".join(missing))
        return False
    hook_registry.register(targets[0], capture_context_graphs, kinds.AROUND)
    return True


def enable_lsa(design: DesignSettings, registry=None, targets: tuple = GROUPED_QUERY_TARGETS,
               graph_targets: tuple = CONTEXT_GRAPH_TARGETS) -> int:
    """Enable the design on this process; returns the hooks registered.

    Raises:
        RuntimeError: A target no longer resolves (nothing is registered then), or the design names no map file.
    """
    if not design.serving.projections:
        raise RuntimeError(f"the model config's {settings.BLOCK!r} names a design with no serving.projections - the "
                           "indexer reads keys and queries through a trained map and there is no index without one")
    missing = unresolved(targets)
    if missing:
        raise RuntimeError("lsa cannot attach to this sglang - these targets no longer resolve: " + "; ".join(missing))
    hook_registry, kinds = _registry(registry)
    by_method = {
        "__init__": (enable, kinds.AFTER),
        "init_forward_metadata": (maintain, kinds.BEFORE),
        "init_forward_metadata_out_graph": (maintain, kinds.BEFORE),
        "forward_extend": (backend.select_and_read, kinds.AROUND),
        "forward_decode": (backend.select_and_read, kinds.AROUND),
    }
    hooks = [(target, *by_method[target.rpartition(".")[2]]) for target in targets]
    for target, hook, kind in hooks:
        hook_registry.register(target, hook, kind)
    ranged = bool(design.serving.decode_context_limits) and context_graphs(hook_registry, kinds, graph_targets)
    hook_registry.apply_hooks()
    ENABLED["design"] = design
    print(f"{BANNER_READY} lsa-top_level{design.indexer.top_level}-decode_{design.serving.decode} width {design.width} "
          f"map {design.serving.projections} kernels {design.serving.kernels}", flush=True)
    logger.info("lsa: %d hooks registered", len(hooks) + ranged)
    return len(hooks) + ranged


def configure(result: None, self: Any, *args: Any, registry=None, **kwargs: Any) -> None:
    """AFTER hook of `ModelConfig.__init__`: read the settings block off the model config and enable its design
    once a process (plugin.py:251-318). A config without the block leaves the server as it was."""
    block = getattr(getattr(self, "hf_config", self), settings.BLOCK, None)
    if block is None or "design" in ENABLED:
        return
    enable_lsa(settings.parse(block), registry=registry)


def register(registry=None) -> None:
    """Carry the plugin's one standing hook, on the model config (plugin.py:991-1010).

    Raises:
        RuntimeError: The model config's constructor no longer resolves.
    """
    if registry is None:
        missing = unresolved((MODEL_CONFIG, HOOK_REGISTRY + ".HookRegistry"))
        if missing:
            raise RuntimeError("lsa cannot read its settings from this sglang - " + "; ".join(missing))
    hook_registry, kinds = _registry(registry)
    hook_registry.register(MODEL_CONFIG, configure, kinds.AFTER)
    logger.info("lsa: settings are read from the model config's %r block", settings.BLOCK)
