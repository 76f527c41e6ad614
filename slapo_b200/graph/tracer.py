"""Hierarchy-preserving graph capture.

``trace(model, ...)`` turns an ``nn.Module`` tree into a tree of
``torch.fx.GraphModule`` objects that has the *same* shape as the module tree:
each level is traced with its direct children (and every element of a child
``ModuleList``) kept as opaque ``call_module`` nodes, and each child is then
traced on its own and re-attached under the same name.  A level that cannot
be traced (data-dependent control flow, ...) is left as the original module
and a warning is logged, so scheduling of the rest of the model goes on.

``flatten=True`` produces a single graph with dotted targets instead.

Three capture engines are selectable by name:

* ``"pytorch"`` - ``torch.fx`` symbolic tracing (default);
* ``"huggingface"`` - meta-tensor propagation in the manner of the tracer that
  ``transformers.utils.fx`` used to ship (it no longer exists): the top level
  is traced on a meta-device copy of the model with dummy meta inputs derived
  from the forward signature and ``config`` (batch 2, ``config["seq_len"]`` or
  16 tokens; integer ids for ``*_ids`` / ``labels`` / ``*mask`` arguments,
  ``[2, seq, hidden_size]`` floats otherwise), every proxy carries the meta
  tensor of its value, so ``x.size()``, ``x.shape[i]`` and Python control flow
  on them resolve to constants; shapes and dtypes stay on the nodes
  (``node.meta["shape"]`` / ``["dtype"]``).  Lower levels of a hierarchical trace
  use the plain engine;
* ``"dynamo"`` - ``torch.export`` capture (always flat).

Parity: slapo/tracer.py:150-272 (hierarchical tracing), :24-25,:511-520
(leaf rule), :275-667 (entry point) of the reference.
"""
from __future__ import annotations

import inspect
import traceback

import torch
from torch import fx, nn

from ..logger import get_logger

logger = get_logger("tracer")


def is_fx_tracing() -> bool:
    """True while an fx symbolic trace is running (works on every torch 2.x)."""
    try:
        from torch.fx._symbolic_trace import is_fx_tracing as _f

        return bool(_f())
    except Exception:  # pragma: no cover
        return False


_OPS_PACKAGE = __name__.split(".")[0] + ".ops."
# ``decompose()`` swaps a Linear for this class precisely so that ``+ bias`` shows up in a graph
_OPS_MEANT_FOR_TRACING = ("LinearWithSeparateBias",)


class HierTracer(fx.Tracer):
    """fx tracer with name/class based leaf rules.

    A module is a leaf when ``module.traceable is False``, when its qualified
    name is listed in ``leaf_modules``, when an entry of ``leaf_modules`` is a
    substring of its class name, or by the stock fx rule (``torch.nn`` layers).
    """

    name = "pytorch"

    def __init__(self, leaf_modules=None, forced_leaf_names=None, keep_ops_whole=True):
        super().__init__(param_shapes_constant=True)
        self.leaf_modules = list(leaf_modules or [])
        self.forced_leaf_names = set(forced_leaf_names or [])
        self.keep_ops_whole = keep_ops_whole

    def user_leaf(self, m: nn.Module, qualname: str) -> bool:
        if getattr(m, "traceable", True) is False:
            return True
        # The operators of this package that a recipe swapped in (attention, fused blocks,
        # norms) stay whole when a level above them is traced: dissolved into a graph, their
        # parameters end up on bare containers (which class-dispatching initialisers do not
        # recognise) and their forward loses the kernel path.  Tracing one of them on its own
        # (``sch[path].trace()``) still works: the rule is about children, and a flattened
        # trace - which asks for everything in one graph - does not apply it.
        if self.keep_ops_whole and type(m).__name__ not in _OPS_MEANT_FOR_TRACING:
            if type(m).__module__.startswith(_OPS_PACKAGE):
                return True
            # Likewise a module that owns parameters itself (a position table, a norm, a head
            # with its own bias): its forward is a primitive of the model, and its class is
            # what an initialiser dispatches on.
            if any(p is not None for p in m._parameters.values()):
                return True
        cls = type(m).__name__
        for pat in self.leaf_modules:
            if isinstance(pat, type):
                if isinstance(m, pat):
                    return True
            elif pat == qualname or (pat and pat in cls):
                return True
        return False

    def is_leaf_module(self, m: nn.Module, module_qualified_name: str) -> bool:
        if module_qualified_name in self.forced_leaf_names:
            return True
        # a forward that reaches past a child (``self.model.decoder(...)``): the grandchild is
        # the unit of this level
        if any(module_qualified_name.startswith(name + ".") for name in self.forced_leaf_names):
            return True
        if self.user_leaf(m, module_qualified_name):
            return True
        if isinstance(m, fx.GraphModule):
            return False
        return super().is_leaf_module(m, module_qualified_name)


_META_TRACER_CLS = []


def MetaHierTracer(leaf_modules=None, forced_leaf_names=None, keep_ops_whole=True):   # noqa: N802
    """The leaf rules of :class:`HierTracer` on ``torch.fx``'s meta-tensor tracer (the class
    is composed on first use, so the experimental module is imported only then)."""
    if not _META_TRACER_CLS:
        from torch.fx.experimental.meta_tracer import MetaTracer

        from torch.fx.experimental.meta_tracer import MetaProxy

        class ShapeProxy(MetaProxy):
            """``ndim`` reads like ``dim()``: a plain int once the meta tensor is known."""

            @property
            def ndim(self):
                return self.dim()

        def proxy(self, node):
            return ShapeProxy(node, self)

        _META_TRACER_CLS.append(type("MetaHierTracer", (HierTracer, MetaTracer), {
            "name": "huggingface", "create_proxy": _meta_create_proxy, "proxy": proxy,
            "call_module": _meta_call_module, "_in_meta_eval": False}))
    return _META_TRACER_CLS[0](leaf_modules, forced_leaf_names, keep_ops_whole)


def _meta_call_module(self, m, forward, args, kwargs):
    # While the output shape of a leaf module is being computed on meta tensors, the modules
    # INSIDE that leaf just run: they must not be recorded as nodes of the graph.
    if self._in_meta_eval:
        return forward(*args, **kwargs)
    from torch.fx.experimental.meta_tracer import MetaTracer

    return MetaTracer.call_module(self, m, forward, args, kwargs)


def _meta_create_proxy(self, kind, target, args, kwargs, name=None, type_expr=None,
                       proxy_factory_fn=None):
    from torch.fx.experimental.meta_tracer import MetaTracer

    self._in_meta_eval = kind == "call_module"
    restore = None
    if kind == "call_module":
        restore = _apply_pre_hook_shapes(self.root, target, args)
    try:
        rv = MetaTracer.create_proxy(self, kind, target, args, kwargs, name, type_expr,
                                     proxy_factory_fn)
    finally:
        self._in_meta_eval = False
        if restore is not None:
            restore[0]._tensor_meta = restore[1]
    if kind == "call_module":
        _apply_post_hook_shapes(self.root, target, rv)
    meta = getattr(rv, "_tensor_meta", None)
    if isinstance(meta, torch.Tensor):
        rv.node.meta["shape"] = tuple(meta.shape)
        rv.node.meta["dtype"] = meta.dtype
    return rv


def _hook_shape_fns(hooks):
    """``meta_shape`` callables of the hooks that have one (``sync`` collectives and the
    vocabulary-parallel embedding hooks): leaf modules run without their hooks while shapes
    are propagated on meta tensors, so the hooks' effect on the token axes - a scatter at the
    start of a sequence-parallel region, the all-gather in front of a column-parallel layer -
    is applied to the recorded shapes instead."""
    out = []
    for hook in hooks.values():
        owner = getattr(hook, "__self__", hook)
        fn = getattr(owner, "meta_shape", None)
        # the embedding hooks are a pre / post pair on one object: the shape changes in post
        if fn is not None and getattr(hook, "__name__", "") != "pre":
            out.append(fn)
    return out


def _leaf_or_none(root, target):
    try:
        return root.get_submodule(target)
    except AttributeError:
        return None


def _apply_pre_hook_shapes(root, target, args):
    mod = _leaf_or_none(root, target)
    first = args[0] if args else None
    meta = getattr(first, "_tensor_meta", None)
    if mod is None or not isinstance(meta, torch.Tensor):
        return None
    shape = tuple(meta.shape)
    for fn in _hook_shape_fns(mod._forward_pre_hooks):
        shape = fn(shape)
    if shape == tuple(meta.shape):
        return None
    first._tensor_meta = meta.new_empty(shape)
    return first, meta


def _apply_post_hook_shapes(root, target, rv):
    mod = _leaf_or_none(root, target)
    meta = getattr(rv, "_tensor_meta", None)
    if mod is None or not isinstance(meta, torch.Tensor):
        return
    shape = tuple(meta.shape)
    for fn in _hook_shape_fns(mod._forward_hooks):
        shape = fn(shape)
    if shape != tuple(meta.shape):
        rv._tensor_meta = meta.new_empty(shape)


_INT_ARG_HINTS = ("ids", "labels", "mask", "positions")
# a level with at most this many parameter elements may be traced on real inputs (see
# _trace_with_meta): embeddings and the like, never a whole trunk
_REAL_RETRACE_LIMIT = 200_000_000


def dummy_meta_inputs(root: nn.Module, concrete_args=None, config=None):
    """Meta tensors for the forward arguments that stay symbolic: what the ``"huggingface"``
    engine propagates.  ``config`` (dict or object) may give ``seq_len``, ``hidden_size``,
    ``batch_size`` and ``input_shapes = {name: (shape, dtype)}`` (or just the shape) for anything
    unusual."""
    get = (lambda k, d=None: config.get(k, d)) if isinstance(config, dict) else \
        (lambda k, d=None: getattr(config, k, d))
    batch, seq = get("batch_size", 2) or 2, get("seq_len", 16) or 16
    hidden = get("hidden_size", None) or get("d_model", None) or get("n_embd", None) or 16
    explicit = get("input_shapes", None) or {}
    metas = {}
    for name, par in inspect.signature(root.forward).parameters.items():
        if par.kind in (par.VAR_POSITIONAL, par.VAR_KEYWORD) or name in (concrete_args or {}):
            continue
        if name in explicit:
            entry = explicit[name]
            if entry and all(isinstance(v, int) for v in entry):      # a bare shape
                entry = (entry, torch.long if any(h in name for h in _INT_ARG_HINTS)
                         else torch.float32)
            shape, dtype = entry
            metas[name] = torch.empty(tuple(shape), dtype=dtype, device="meta")
        elif par.default is not inspect.Parameter.empty:
            continue            # optional and not named: frozen at its default by the caller
        elif any(h in name for h in _INT_ARG_HINTS):
            metas[name] = torch.empty((batch, seq), dtype=torch.long, device="meta")
        else:
            metas[name] = torch.empty((batch, seq, hidden), dtype=torch.float32, device="meta")
    if not metas:
        # Hugging Face models declare every input optional (``input_ids=None``): keep the
        # token ids live (and the decoder's for encoder-decoder models), freeze the rest
        params = inspect.signature(root.forward).parameters
        frozen = concrete_args or {}
        for name in ("input_ids", "decoder_input_ids"):
            if name in params and name not in frozen and (
                    name == "input_ids" or get("is_encoder_decoder", False)):
                metas[name] = torch.empty((batch, seq), dtype=torch.long, device="meta")
    return metas


class _fixed_signature:
    """Context manager: while active, ``root``'s class is a subclass whose ``forward`` has the
    named parameters of the original one but neither ``*args`` nor ``**kwargs``.

    fx makes one placeholder per parameter of ``type(root).forward`` and then calls it with
    those placeholders; a ``**kwargs`` placeholder is a Proxy that the call tries to unpack
    ("Proxy object cannot be iterated").  Hugging Face modules carry a catch-all ``**kwargs``
    on almost every forward; nothing is passed through it in a training graph, so it is
    dropped for the trace."""

    def __init__(self, root):
        self.root = root
        self.orig_cls = None

    def __enter__(self):
        root = self.root
        try:
            sig = inspect.signature(type(root).forward)
        except (TypeError, ValueError):
            return self
        params = list(sig.parameters.values())
        if not any(p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD) for p in params):
            return self
        named = [p for p in params[1:] if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD,
                                                     p.KEYWORD_ONLY)]
        defaults = {}
        decl, call = [], []
        for p in named:
            if p.default is inspect.Parameter.empty:
                decl.append(p.name)
            else:
                defaults[p.name] = p.default
                decl.append(f"{p.name}=__defaults[{p.name!r}]")
            # by keyword: decorators that wrap a forward as (*args, **kwargs) and fill in
            # keyword defaults of their own must not collide with positional values
            call.append(p.name if p.kind == p.POSITIONAL_ONLY else f"{p.name}={p.name}")
        src = (f"def forward(self, {', '.join(decl)}):\n"
               f"    return __orig(self, {', '.join(call)})\n")
        scope = {"__orig": type(root).forward, "__defaults": defaults}
        exec(src, scope)   # noqa: S102 - source built from parameter names only
        self.orig_cls = type(root)
        sub = type(self.orig_cls.__name__, (self.orig_cls,), {"forward": scope["forward"]})
        sub.__module__ = self.orig_cls.__module__
        sub.__qualname__ = self.orig_cls.__qualname__
        root.__class__ = sub
        return self

    def __exit__(self, *exc):
        if self.orig_cls is not None:
            self.root.__class__ = self.orig_cls
        return False


def _direct_child_names(root: nn.Module):
    names = []
    for key, child in root.named_children():
        if isinstance(child, nn.ModuleList):
            names += [f"{key}.{sub}" for sub, _ in child.named_children()]
        else:
            names.append(key)
    return names


def _fill_concrete_args(root, concrete_args, call_node):
    """Values to specialise the trace of ``root`` on.

    Top level: the user's ``concrete_args``.  Lower levels: every forward
    parameter that the parent's call site does not bind and that has a
    default is frozen at that default, so an optional input that is never
    passed does not turn into a required placeholder."""
    if call_node is None:
        return dict(concrete_args or {})
    sig = inspect.signature(root.forward)
    params = [p for p in sig.parameters.values()
              if p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD)]
    bound = dict(zip((p.name for p in params), call_node.args))
    bound.update(call_node.kwargs)
    frozen = {}
    for p in params:
        if p.name in bound:
            val = bound[p.name]
            if val is None or isinstance(val, bool):
                frozen[p.name] = val  # the call site passes a literal
        elif p.default is not inspect.Parameter.empty:
            frozen[p.name] = p.default
    return frozen


def _strip_specialisation_guards(graph: fx.Graph, frozen: dict):
    """fx keeps a placeholder ``<name>_1`` plus an assert for every frozen
    argument.  Give the placeholder its original name back (so keyword calls
    keep working) and drop the guards, which would otherwise run on every
    forward."""
    if not frozen:
        return
    for node in list(graph.nodes):
        if node.op != "placeholder":
            continue
        base = node.target[:-2] if node.target.endswith("_1") else None
        if base not in frozen:
            continue
        node.target = base
        work = list(node.users)
        while work:
            user = work.pop()
            if user.op == "call_function" and (
                    user.target is torch._assert
                    or getattr(user.target, "__name__", "") == "_assert_is_none"):
                graph.erase_node(user)
            elif user.op == "call_function" and all(
                    u.op == "call_function" and (u.target is torch._assert) for u in user.users):
                for u in list(user.users):
                    graph.erase_node(u)
                graph.erase_node(user)


def _adapt_call_site(node: fx.Node, child: fx.GraphModule):
    """Make the parent's call of a freshly traced child fit the child's graph.

    * Keyword arguments that the traced child no longer takes (its catch-all ``**kwargs`` was
      dropped for the trace: Hugging Face's ``return_dict`` and friends) are removed.
    * A Hugging Face ``ModelOutput`` becomes a plain dict in the child's graph.  The parent
      written against ``ModelOutput`` reads it by position (``outputs[0]``: the k-th entry that
      is not None) or by attribute (``outputs.last_hidden_state``); both are rewritten to the
      dict key."""
    import builtins
    import operator

    names = {str(n.target).lstrip("*") for n in child.graph.nodes if n.op == "placeholder"}
    if any(k not in names for k in node.kwargs):
        node.kwargs = {k: v for k, v in node.kwargs.items() if k in names}
    out = next((n for n in child.graph.nodes if n.op == "output"), None)
    ret = out.args[0] if out is not None and out.args else None
    if not isinstance(ret, dict):
        return
    present = [k for k, v in ret.items() if v is not None]
    for user in list(node.users):
        if user.op != "call_function" or not user.args or user.args[0] is not node:
            continue
        if user.target is operator.getitem and isinstance(user.args[1], int):
            idx = user.args[1]
            if -len(present) <= idx < len(present):
                user.args = (node, present[idx])
        elif user.target is builtins.getattr and isinstance(user.args[1], str):
            if user.args[1] in ret:
                user.target = operator.getitem
            elif not hasattr(dict, user.args[1]):
                # a field the child did not produce reads as None on a ModelOutput
                user.args = (node, user.args[1], None)


def _get_submodule_or_none(root, target):
    cur = root
    for tok in target.split("."):
        if not hasattr(cur, tok):
            return None
        cur = getattr(cur, tok)
    return cur


def _metas_from_call(root, call_node):
    """Meta tensors for the arguments of a child module, taken from the shapes that the
    parent's meta-tensor trace recorded on the nodes of the call site; ``None`` when an
    argument is a node without a recorded tensor shape (then the plain engine runs)."""
    sig = inspect.signature(root.forward)
    params = [p for p in sig.parameters.values()
              if p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD)]
    bound = dict(zip((p.name for p in params), call_node.args))
    bound.update({k: v for k, v in call_node.kwargs.items() if k in sig.parameters})
    metas = {}
    for name, val in bound.items():
        if isinstance(val, fx.Node):
            if "shape" not in val.meta:
                return None
            metas[name] = torch.empty(val.meta["shape"], dtype=val.meta["dtype"], device="meta")
    return metas or None


def _trace_with_meta(root, leaf_modules, forced, cargs, config, metas=None):
    """The ``"huggingface"`` engine: trace a meta-device copy (so that leaf modules can run on
    the meta inputs) and return its graph, whose targets are names and therefore fit the real
    module tree just as well.  ``metas``: the inputs of a lower level (from the parent's call
    site); at the top they are made up from the signature."""
    import copy

    if metas is None:
        metas = dummy_meta_inputs(root, cargs, config)
    frozen = dict(cargs)
    for name, par in inspect.signature(root.forward).parameters.items():
        if name not in metas and name not in frozen and par.default is not inspect.Parameter.empty:
            frozen[name] = par.default
    if frozen.get("use_cache", False) is None:
        # Hugging Face decoders build a key / value cache object when ``use_cache`` is left to
        # the configuration; a training graph has none
        frozen["use_cache"] = False
    try:
        shadow = copy.deepcopy(root).to("meta")
    except Exception:       # modules that cannot be copied are traced in place
        shadow = root
    tracer = MetaHierTracer(leaf_modules, forced, bool(forced))
    with _fixed_signature(shadow):
        graph = tracer.trace(shadow, meta_args=metas, concrete_args=frozen or None)
    if any(node.op == "get_attr" and _get_submodule_or_none(root, node.target) is None
           for node in graph.nodes):
        # A tensor built inside forward (a slice of a buffer, say) becomes an attribute of the
        # traced root - here the meta copy, whose tensors have no values.  A small level on a
        # real device is traced again IN PLACE on real zero-filled inputs of the same shapes:
        # the constants then carry values and land on the real module.
        n_elems = sum(p.numel() for p in root.parameters())
        device = next((p.device for p in root.parameters()), torch.device("cpu"))
        if shadow is root or device.type == "meta" or n_elems > _REAL_RETRACE_LIMIT:
            raise RuntimeError("a tensor constant was created during the meta trace")
        reals = {k: torch.zeros(v.shape, dtype=v.dtype, device=device) for k, v in metas.items()}
        tracer = MetaHierTracer(leaf_modules, forced, bool(forced))
        with _fixed_signature(root), torch.no_grad():
            graph = tracer.trace(root, meta_args=reals, concrete_args=frozen or None)
    return graph, frozen


def _trace_level(root: nn.Module, *, leaf_modules, flatten, recursive, concrete_args,
                 call_node=None, engine="pytorch", config=None):
    if isinstance(root, fx.GraphModule):
        return root
    whole = not flatten
    judge = MetaHierTracer(leaf_modules, None, whole) if engine == "huggingface" \
        else HierTracer(leaf_modules, None, whole)
    forced = [] if flatten else _direct_child_names(root)
    tracer = HierTracer(leaf_modules, forced, whole)
    graph = None
    cargs = _fill_concrete_args(root, concrete_args, call_node)
    metas = None
    if engine == "huggingface" and call_node is not None:
        metas = _metas_from_call(root, call_node)
    if engine == "huggingface" and (call_node is None or metas is not None):
        try:
            graph, cargs = _trace_with_meta(root, leaf_modules, forced, cargs, config, metas)
        except Exception as meta_err:
            logger.info("meta-tensor trace of %s failed (%s); trying the plain engine",
                        type(root).__name__, meta_err)
            graph = None
    try:
        if graph is None:
            with _fixed_signature(root):
                graph = tracer.trace(root, concrete_args=cargs or None)
    except Exception as first_err:
        # Optional inputs (default None) that steer Python control flow cannot
        # stay symbolic.  Retry once with every such input frozen at None; the
        # caller names the ones it needs live through concrete_args.
        sig = inspect.signature(root.forward)
        optional = {n: None for n, p in sig.parameters.items()
                    if p.default is None and n not in cargs}
        if optional and call_node is None:
            try:
                cargs = dict(cargs, **optional)
                with _fixed_signature(root):
                    graph = HierTracer(leaf_modules, forced, whole).trace(root, concrete_args=cargs)
                logger.info("traced %s with optional inputs %s frozen at None",
                            type(root).__name__, sorted(optional))
            except Exception:
                graph = None
        if graph is None:
            err = first_err
    if graph is None:  # untraceable level: keep the eager module
        err = locals().get("err", "unknown error")
        logger.debug(traceback.format_exc())
        logger.warning("cannot trace %s (%s); left as an eager module",
                       type(root).__name__, err)
        return root

    _strip_specialisation_guards(graph, cargs)
    for node in graph.nodes:
        # a child module literally called "self" (Hugging Face attention blocks)
        # would shadow the module reference in the generated forward
        if node.name == "self" and node.op != "placeholder":
            if hasattr(node, "_rename"):
                node._rename("self_mod")
            else:  # pragma: no cover - older fx
                node.name = "self_mod"
    if flatten:
        gm = fx.GraphModule(root, graph, class_name=type(root).__name__)
    else:
        pieces = {}
        for node in graph.nodes:
            if node.op == "call_module":
                child = _get_submodule_or_none(root, node.target)
                qual = node.target
                if (recursive and child is not None and not judge.user_leaf(child, qual)
                        and not fx.Tracer.is_leaf_module(judge, child, qual)):
                    eager = child
                    child = _trace_level(
                        child, leaf_modules=leaf_modules, flatten=False, recursive=True,
                        concrete_args=concrete_args, call_node=node, engine=engine,
                        config=config)
                    if child is not eager:
                        # the traced child stands in for the eager one: its hooks (the
                        # collectives that ``sync`` registered among them) move along
                        from ..utils.common import transfer_hooks

                        transfer_hooks(eager, child)
                    if isinstance(child, fx.GraphModule):
                        _adapt_call_site(node, child)
                pieces[node.target] = child
            elif node.op == "get_attr":
                pieces[node.target] = _get_submodule_or_none(root, node.target)
        gm = fx.GraphModule(pieces, graph, class_name=type(root).__name__)
        for target in pieces:
            # "model.decoder" as a call target: fx made a bare module "model" to hold it;
            # the schedule tree walks through such containers to the traced grandchild
            tokens = target.split(".")
            for depth in range(1, len(tokens)):
                holder = _get_submodule_or_none(gm, ".".join(tokens[:depth]))
                if type(holder) is nn.Module:
                    holder.schedule_container = True
    gm.graph.eliminate_dead_code()
    gm.delete_all_unused_submodules()
    gm.graph.lint()
    gm.recompile()
    # keep plain-data attributes (configs, flags) that schedules may read later
    for key, val in vars(root).items():
        if key.startswith("_") or key in ("training",) or hasattr(gm, key):
            continue
        if isinstance(val, (int, float, str, bool, tuple)) or val is None:
            try:
                setattr(gm, key, val)
            except Exception:  # pragma: no cover
                pass
    gm.train(root.training)
    _keep_buffer_persistence(root, gm)
    return gm


def _keep_buffer_persistence(root, gm):
    """``fx.GraphModule`` registers the buffers it copies as persistent; a buffer that the
    eager module kept out of its ``state_dict`` (``persistent=False``: position ids, causal
    masks) stays out of the traced module's as well."""
    eager = dict(root.named_modules())
    for path, mod in gm.named_modules():
        src = eager.get(path)
        if src is None or src is mod:
            continue
        for name in getattr(src, "_non_persistent_buffers_set", ()):
            if name in mod._buffers:
                mod._non_persistent_buffers_set.add(name)


def _trace_dynamo(root, concrete_args):
    """``torch.export`` capture.  ``concrete_args`` holds the example inputs: either under the
    key ``"example_inputs"`` (a tuple of positional arguments) or, as in the reference
    (slapo/tracer.py:642-659), one entry per forward argument."""
    concrete_args = dict(concrete_args or {})
    if not concrete_args:
        raise ValueError('the "dynamo" tracer needs example inputs in concrete_args')
    if "example_inputs" in concrete_args:
        args, kwargs = tuple(concrete_args["example_inputs"]), {}
    else:
        args, kwargs = (), concrete_args
    try:
        device = next(root.parameters()).device
    except StopIteration:
        device = None
    move = lambda v: v.to(device) if isinstance(v, torch.Tensor) and device is not None else v
    exported = torch.export.export(root, tuple(move(a) for a in args),
                                   {k: move(v) for k, v in kwargs.items()}, strict=False)
    captured = exported.module()
    # The exported module refuses train() / eval(); an ordinary GraphModule over the same
    # graph and attributes behaves like every other traced module of the schedule.
    gm = fx.GraphModule(captured, captured.graph)
    gm.train(root.training)
    return gm


def trace(model: nn.Module, tracer: str = "pytorch", recursive: bool = True,
          flatten: bool = False, leaf_modules=None, concrete_args=None, config=None,
          **_unused):
    """Capture ``model`` as a (tree of) GraphModule(s); see the module docstring.

    Returns the original module unchanged when the top level cannot be traced.
    """
    if not isinstance(tracer, str):
        raise NotImplementedError("custom tracer classes are not supported; pass a name")
    if tracer == "dynamo":
        return _trace_dynamo(model, concrete_args)
    if tracer not in ("pytorch", "huggingface"):
        raise ValueError(f"unknown tracer {tracer}")
    return _trace_level(
        model, leaf_modules=list(leaf_modules or []), flatten=flatten, recursive=recursive,
        concrete_args=concrete_args, engine=tracer, config=config)


trace_module = trace
