"""FX graph -> ``DecoderProgram``: recognise the decoder the captured ATen graph spells out.

The reference lowers every ATen op into a generic tensor-program IR and forms regions by
recogniser (``src/megabake/ops/{gemm,norm,rope,elementwise,attention}.py``,
``src/megabake/regions.py:15-37``).  This backend covers the decoder op set only, so it matches
the post-AOT graph directly, walking backwards from the logits:

    logits  <- linear(rmsnorm(h_L), lm_head)
    h_l     <- add(h_mid, linear(gated(linear(n2), linear(n2)), down)),  n2 = rmsnorm(h_mid)
    h_mid   <- add(h_in, linear(kv_attention(rope(q), rope(k), v, caches, length), o_proj))
               q, k, v = linear(rmsnorm(h_in), ...)
    h_0     <- embedding(ids) [* scale]

What is kept of each pattern is exactly what fixes a rounding point of the eager forward (which
norm spelling, bias inside the GEMM, which activation, the extra query scale); everything else
(views, reshapes, permutes that only move size-1 axes, contiguity clones) is skipped as layout
noise.  Anything that does not fit raises ``CompilerError(stage="pattern-recognition")``: there
is no second compiler to fall back to.
"""

from __future__ import annotations

import math
import operator
from collections import Counter
from dataclasses import dataclass

import torch

from .diagnostics import fail
from .program import DecoderProgram, LayerBinding

aten = torch.ops.aten
prims = torch.ops.prims

_VIEW_TARGETS = {
    aten.view.default, aten.reshape.default, aten._unsafe_view.default, aten.unsqueeze.default,
    aten.squeeze.dim, aten.squeeze.default, aten.expand.default, aten.clone.default,
    aten.alias.default, aten.permute.default, aten.transpose.int, aten.slice.Tensor,
    aten.contiguous.default, aten.detach.default,
}


def _val(node):
    return node.meta.get("val") if hasattr(node, "meta") else None


def _shape(node) -> tuple[int, ...]:
    val = _val(node)
    return tuple(val.shape) if isinstance(val, torch.Tensor) else ()


def _dense(shape) -> tuple[int, ...]:
    return tuple(d for d in shape if d != 1)


def _is(node, *targets) -> bool:
    return isinstance(node, torch.fx.Node) and node.op == "call_function" and node.target in targets


# Prefill graphs move the head axis in front of the token axis for RoPE and back again for the
# attention operator ([B, T, H, D] <-> [B, H, T, D]).  While a prefill graph is matched these
# transposes count as layout-only: the operands are identified by the projection they come
# from, and the attention call is checked to receive them as [B, T, H, D] again.
_HEAD_TOKEN_SWAPS_ARE_LAYOUT = False


def _keeps_order(node) -> bool:
    """True if a view-like op leaves the element order untouched (it only reshapes, adds or
    moves size-1 axes, or copies)."""
    source = node.args[0]
    if not isinstance(source, torch.fx.Node):
        return False
    if node.target in (aten.view.default, aten.reshape.default, aten._unsafe_view.default):
        return True  # a reshape never reorders the (row-major) elements
    if math.prod(_shape(node)) != math.prod(_shape(source)):
        return False  # a broadcasting expand or a partial slice
    if node.target in (aten.permute.default, aten.transpose.int):
        shape = _shape(source)
        if node.target is aten.permute.default:
            order = [d % len(shape) for d in node.args[1]]
        else:
            order = list(range(len(shape)))
            a, b = node.args[1] % len(shape), node.args[2] % len(shape)
            order[a], order[b] = order[b], order[a]
        moved = [d for d in order if shape[d] != 1]
        if _HEAD_TOKEN_SWAPS_ARE_LAYOUT and len(shape) == 4 and order == [0, 2, 1, 3]:
            return True
        return moved == sorted(moved)
    return True


def strip(node):
    """Skip layout-only ops."""
    while _is(node, *_VIEW_TARGETS) and _keeps_order(node):
        node = node.args[0]
    return node


def _placeholder_index(node, order: dict) -> int | None:
    node = strip(node)
    if isinstance(node, torch.fx.Node) and node.op == "placeholder":
        return order[node]
    return None


def _convert(node, dtype):
    """``convert_element_type(x, dtype)`` -> x, else None."""
    node = strip(node)
    if _is(node, prims.convert_element_type.default, aten._to_copy.default):
        target = node.args[1] if len(node.args) > 1 else node.kwargs.get("dtype")
        if target == dtype:
            return node.args[0]
    return None


def _binary(node, target):
    node = strip(node)
    if _is(node, target) and len(node.args) >= 2:
        return node.args[0], node.args[1]
    return None


def _scalar(value) -> float | None:
    return float(value) if isinstance(value, (int, float)) and not isinstance(value, bool) else None


@dataclass
class Linear:
    node: torch.fx.Node
    x: torch.fx.Node  # stripped activation node
    weight: int
    bias: int | None
    out_features: int
    in_features: int


class _Matcher:
    def __init__(self, graph: torch.fx.Graph):
        self.graph = graph
        placeholders = [n for n in graph.nodes if n.op == "placeholder"]
        self.order = {node: index for index, node in enumerate(placeholders)}
        self.placeholders = placeholders

    def refuse(self, what: str, node=None):
        names = (node.name,) if isinstance(node, torch.fx.Node) else ()
        fail("pattern-recognition", f"the captured graph is not a decoder this backend covers: {what}",
             requirement="Llama / Qwen2 / Gemma style pre-norm decoder over megabake::kv_attention",
             ops=names)

    # -- linear -------------------------------------------------------------------------
    def linear(self, node) -> Linear | None:
        node = strip(node)
        bias = None
        if _is(node, aten.mm.default):
            x, wt = node.args
        elif _is(node, aten.addmm.default):
            bias_node, x, wt = node.args[:3]
            bias = _placeholder_index(bias_node, self.order)
            if bias is None:
                return None
        else:
            return None
        if not _is(wt, aten.permute.default, aten.t.default, aten.transpose.int):
            return None
        weight = wt.args[0]
        if not (isinstance(weight, torch.fx.Node) and weight.op == "placeholder"):
            return None
        out_features, in_features = _shape(weight)
        return Linear(node, strip(x), self.order[weight], bias, out_features, in_features)

    # -- rmsnorm --------------------------------------------------------------------------
    def _normalised(self, node):
        """``x32 * rsqrt(mean(x32 ** 2, -1, keepdim) + eps)`` -> (x, eps)."""
        pair = _binary(node, aten.mul.Tensor)
        if pair is None:
            return None
        for wide, scale in (pair, pair[::-1]):
            if not _is(strip(scale), aten.rsqrt.default):
                continue
            inner = _binary(strip(scale).args[0], aten.add.Tensor)
            if inner is None or _scalar(inner[1]) is None:
                continue
            mean = strip(inner[0])
            if not _is(mean, aten.mean.dim):
                continue
            power = strip(mean.args[0])
            if not (_is(power, aten.pow.Tensor_Scalar) and power.args[1] == 2):
                continue
            if strip(power.args[0]) is not strip(wide):
                continue
            x = _convert(wide, torch.float32)
            if x is None:
                continue
            return strip(x), float(inner[1])
        return None

    def rmsnorm(self, node):
        """-> (x, weight placeholder, eps, kind) or None."""
        node = strip(node)
        pair = _binary(node, aten.mul.Tensor)
        if pair is not None:  # Llama spelling: weight * bf16(normalised)
            for weight, body in (pair, pair[::-1]):
                index = _placeholder_index(weight, self.order)
                if index is None:
                    continue
                inner = _convert(body, torch.bfloat16)
                found = self._normalised(inner) if inner is not None else None
                if found is not None:
                    return found[0], index, found[1], "llama"
        inner = _convert(node, torch.bfloat16)
        if inner is not None:  # Gemma spelling: bf16(normalised * (1 + w32))
            pair = _binary(inner, aten.mul.Tensor)
            if pair is not None:
                for body, gain in (pair, pair[::-1]):
                    plus = _binary(gain, aten.add.Tensor)
                    if plus is None or _scalar(plus[1]) != 1.0:
                        continue
                    weight = _convert(plus[0], torch.float32)
                    index = _placeholder_index(weight, self.order) if weight is not None else None
                    found = self._normalised(body)
                    if index is not None and found is not None:
                        return found[0], index, found[1], "gemma"
        return None

    # -- gated activation -----------------------------------------------------------------
    def _cone(self, node, stop):
        """Operator multiset and scalar constants between ``node`` and ``stop``."""
        ops, constants, seen = Counter(), set(), set()
        stack = [node]
        while stack:
            current = stack.pop()
            if not isinstance(current, torch.fx.Node):
                value = _scalar(current)
                if value is not None:
                    constants.add(value)
                continue
            if current is stop or current in seen:
                continue
            seen.add(current)
            if current.op != "call_function":
                return None
            if current.target not in _VIEW_TARGETS:
                ops[current.target] += 1
            stack.extend(current.args)
        return ops, constants

    def gated(self, node):
        """``act(gate) * up`` -> (gate linear, up linear, activation name) or None."""
        pair = _binary(node, aten.mul.Tensor)
        if pair is None:
            return None
        for activated, up in (pair, pair[::-1]):
            up_linear = self.linear(up)
            inner = _convert(activated, torch.bfloat16)
            if up_linear is None or inner is None:
                continue
            # find the fp32 widening of the gate projection below the activation
            widened = [n for n in self._ancestors(inner)
                       if _is(n, prims.convert_element_type.default, aten._to_copy.default)
                       and self.linear(n.args[0]) is not None]
            if len(widened) != 1:
                continue
            gate_linear = self.linear(widened[0].args[0])
            cone = self._cone(inner, widened[0])
            if cone is None:
                continue
            ops, constants = cone
            if ops == Counter({aten.neg.default: 1, aten.exp.default: 1, aten.add.Tensor: 1,
                               aten.div.Tensor: 1}) and constants == {1.0}:
                return gate_linear, up_linear, "silu"
            if (ops == Counter({aten.mul.Tensor: 6, aten.add.Tensor: 2, aten.tanh.default: 1})
                    and {0.5, 0.044715, 1.0} <= constants
                    and any(abs(c - 0.7978845608028654) < 1e-9 for c in constants)):
                return gate_linear, up_linear, "gelu_tanh"
        return None

    def _ancestors(self, node, limit: int = 64):
        seen, stack, out = set(), [node], []
        while stack and len(out) < limit:
            current = stack.pop()
            if not isinstance(current, torch.fx.Node) or current in seen:
                continue
            seen.add(current)
            out.append(current)
            if current.op == "call_function" and not _is(current, aten.mm.default, aten.addmm.default):
                stack.extend(a for a in current.args if isinstance(a, torch.fx.Node))
        return out

    # -- rotary embedding -------------------------------------------------------------------
    def _table(self, node):
        """A cos/sin table operand -> ("cos" | "sin", scale, inv_freq index, position index)."""
        node = strip(node)
        # StatefulSmolLM-style spelling slices the expanded table; look through that too
        while _is(node, aten.slice.Tensor, aten.expand.default, aten.unsqueeze.default,
                  aten.view.default, aten.clone.default):
            node = node.args[0]
        body = _convert(node, torch.bfloat16)
        if body is None:
            return None
        body = strip(body)
        scale = 1.0
        if _is(body, aten.mul.Tensor) and _scalar(body.args[1]) is not None:
            scale = float(body.args[1])
            body = strip(body.args[0])
        if _is(body, aten.cos.default):
            kind = "cos"
        elif _is(body, aten.sin.default):
            kind = "sin"
        else:
            return None
        # the angles must come from inv_freq (x) position_ids and nothing else
        allowed = _VIEW_TARGETS | {aten.bmm.default, aten.cat.default, aten.mul.Tensor,
                                   prims.convert_element_type.default, aten._to_copy.default}
        leaves, stack, seen = set(), [body.args[0]], set()
        counted_positions = False  # positions 0..T-1 built inside the graph (prefill)
        while stack:
            current = stack.pop()
            if isinstance(current, (list, tuple)):
                stack.extend(current)
                continue
            if not isinstance(current, torch.fx.Node) or current in seen:
                continue
            seen.add(current)
            if current.op == "placeholder":
                leaves.add(current)
            elif _is(current, prims.iota.default):
                if (current.kwargs.get("start", 0) != 0 or current.kwargs.get("step", 1) != 1
                        or counted_positions):
                    return None
                counted_positions = True
            elif _is(current, aten.add.Tensor) and _scalar(current.args[1]) == 0.0:
                stack.append(current.args[0])
            elif current.op == "call_function" and current.target in allowed:
                stack.extend(current.args)
            else:
                return None
        inv = [n for n in leaves if _val(n).dtype.is_floating_point]
        pos = [n for n in leaves if not _val(n).dtype.is_floating_point]
        if len(inv) != 1 or len(pos) + int(counted_positions) != 1:
            return None
        return kind, scale, self.order[inv[0]], (self.order[pos[0]] if pos else None)

    def rope(self, node):
        """Rotary embedding of a projection -> (linear, tables dict) or None.  Covers the
        Hugging Face spelling ``x * cos + cat(-x[half:], x[:half]) * sin`` and the spelling
        with explicit halves ``cat(x1 * c - x2 * s, x2 * c + x1 * s)``."""
        node = strip(node)
        pair = _binary(node, aten.add.Tensor)
        if pair is not None:
            for first, second in (pair, pair[::-1]):
                a, b = _binary(first, aten.mul.Tensor) or (None, None), \
                    _binary(second, aten.mul.Tensor) or (None, None)
                if a[0] is None or b[0] is None:
                    continue
                for x, cos in (a, a[::-1]):
                    for rotated, sin in (b, b[::-1]):
                        tc, ts = self._table(cos), self._table(sin)
                        projection = self.linear(x)
                        if not (tc and ts and projection) or tc[0] != "cos" or ts[0] != "sin":
                            continue
                        if self._is_rotate_half(rotated, projection):
                            return projection, tc, ts
        if _is(node, aten.cat.default) and len(node.args[0]) == 2:
            low, high = node.args[0]
            low_pair, high_pair = _binary(low, aten.sub.Tensor), _binary(high, aten.add.Tensor)
            if low_pair and high_pair:
                first = _binary(low_pair[0], aten.mul.Tensor)
                if first:
                    for x, cos in (first, first[::-1]):
                        projection = self._through_slice(x)
                        tc = self._table(cos)
                        if projection is not None and tc and tc[0] == "cos":
                            other = _binary(low_pair[1], aten.mul.Tensor)
                            ts = None
                            for candidate in other or ():
                                found = self._table(candidate)
                                if found and found[0] == "sin":
                                    ts = found
                            if ts:
                                return projection, tc, ts
        return None

    def _through_slice(self, node):
        node = strip(node)
        while _is(node, aten.slice.Tensor):
            node = strip(node.args[0])
        return self.linear(node)

    def _is_rotate_half(self, node, projection: Linear) -> bool:
        node = strip(node)
        if not (_is(node, aten.cat.default) and len(node.args[0]) == 2):
            return False
        negated, kept = node.args[0]
        negated = strip(negated)
        if not _is(negated, aten.neg.default):
            return False
        upper, lower = strip(negated.args[0]), strip(kept)
        if not (_is(upper, aten.slice.Tensor) and _is(lower, aten.slice.Tensor)):
            return False
        same = (self.linear(upper.args[0]) is not None and self.linear(lower.args[0]) is not None
                and self.linear(upper.args[0]).node is projection.node
                and self.linear(lower.args[0]).node is projection.node)
        half = _shape(upper)[-1]
        return same and upper.args[2] == half and lower.args[2] == 0

    # -- attention ----------------------------------------------------------------------------
    def kv_attention(self, node):
        """The stateful attention call whose result ``node`` is -> dict or None."""
        node = strip(node)
        call = None
        if _is(node, operator.getitem) and node.args[1] == 0:
            call = node.args[0]
        target = torch.ops.megabake.kv_attention.default
        if _is(node, target):
            names = ("source", "key", "value", "key_cache", "value_cache", "valid_length")
            operands = dict(zip(names, node.args))
            state = [operands[n] for n in names[3:]]
        elif (isinstance(call, torch.fx.Node) and call.op == "call_function"
              and "functionaliz" in type(call.target).__name__.lower() and call.args
              and call.args[0] is target):
            operands = call.kwargs
            bases = operands["_all_bases"]
            state = [bases[operands[f"_{n}_base_index"]]
                     for n in ("key_cache", "value_cache", "valid_length")]
        else:
            return None
        indices = [_placeholder_index(n, self.order) for n in state]
        if any(i is None for i in indices):
            self.refuse("KV state tensors must be graph inputs", node)
        return {"source": operands["source"], "key": operands["key"], "value": operands["value"],
                "key_cache": indices[0], "value_cache": indices[1], "valid_length": indices[2]}

    def prefill_attention(self, node):
        """``megabake::attention(q, k, v, mask, scale)`` whose result ``node`` is -> dict."""
        node = strip(node)
        if not _is(node, torch.ops.megabake.attention.default):
            return None
        query, key, value, mask, scale = node.args[:5]
        return {"source": query, "key": key, "value": value, "mask": mask, "scale": float(scale),
                "key_cache": -1, "value_cache": -1, "valid_length": -1, "node": node}

    def prefill_state_attention(self, node):
        """``megabake::prefill_kv_attention`` (causal prefill that also fills the decode state)
        whose result ``node`` is -> dict or None."""
        node = strip(node)
        call = node.args[0] if _is(node, operator.getitem) and node.args[1] == 0 else None
        target = torch.ops.megabake.prefill_kv_attention.default
        if _is(node, target):
            names = ("query", "key", "value", "key_cache", "value_cache", "valid_length", "scale")
            operands = dict(zip(names, node.args))
            state = [operands[n] for n in names[3:6]]
        elif (isinstance(call, torch.fx.Node) and call.op == "call_function"
              and "functionaliz" in type(call.target).__name__.lower() and call.args
              and call.args[0] is target):
            operands = call.kwargs
            bases = operands["_all_bases"]
            state = [bases[operands[f"_{n}_base_index"]]
                     for n in ("key_cache", "value_cache", "valid_length")]
        else:
            return None
        indices = [_placeholder_index(n, self.order) for n in state]
        if any(i is None for i in indices):
            self.refuse("KV state tensors must be graph inputs", node)
        return {"source": operands["query"], "key": operands["key"], "value": operands["value"],
                "mask": None, "causal": True, "scale": float(operands["scale"]), "node": node,
                "key_cache": indices[0], "value_cache": indices[1], "valid_length": indices[2]}

    def constant(self, node, module: torch.fx.GraphModule):
        """Evaluate a sub-graph that depends on no graph input (the mask of a prefill)."""
        memo: dict = {}

        def run(current):
            if isinstance(current, (list, tuple)):
                return type(current)(run(item) for item in current)
            if not isinstance(current, torch.fx.Node):
                return current
            if current in memo:
                return memo[current]
            if current.op == "get_attr":
                value = getattr(module, current.target)
            elif current.op == "call_function":
                value = current.target(*run(current.args),
                                       **{k: run(v) for k, v in current.kwargs.items()})
            else:
                self.refuse("the attention mask depends on a runtime input; call the model "
                            "without attention_mask (a full causal prefill)", current)
            memo[current] = value
            return value

        # recognition runs inside the compiler's tracing modes (fake tensors); the constant has
        # to be computed for real
        from torch.utils._python_dispatch import _disable_current_modes

        with _disable_current_modes(), torch.no_grad():
            return run(node)

    # -- embedding ----------------------------------------------------------------------------
    def embedding(self, node):
        """-> (weight index, ids index, scale placeholder index or None) or None."""
        node = strip(node)
        scale = None
        pair = _binary(node, aten.mul.Tensor)
        if pair is not None:
            for body, factor in (pair, pair[::-1]):
                index = _placeholder_index(factor, self.order)
                if index is not None and _is(strip(body), aten.embedding.default):
                    node, scale = strip(body), index
        if not _is(node, aten.embedding.default):
            return None
        weight = _placeholder_index(node.args[0], self.order)
        ids = _placeholder_index(node.args[1], self.order)
        if weight is None or ids is None:
            return None
        return weight, ids, scale


def recognize_decoder(graph_module: torch.fx.GraphModule, mode: str) -> DecoderProgram:
    """Match the whole graph; raises ``CompilerError`` if it is not a covered decoder."""
    global _HEAD_TOKEN_SWAPS_ARE_LAYOUT
    prefill_ops = (torch.ops.megabake.attention.default,
                   torch.ops.megabake.prefill_kv_attention.default)
    _HEAD_TOKEN_SWAPS_ARE_LAYOUT = any(
        _is(node, *prefill_ops) or (node.op == "call_function" and node.args
                                    and node.args[0] in prefill_ops)
        for node in graph_module.graph.nodes)
    try:
        return _recognize(graph_module, mode)
    finally:
        _HEAD_TOKEN_SWAPS_ARE_LAYOUT = False


def _recognize(graph_module: torch.fx.GraphModule, mode: str) -> DecoderProgram:
    m = _Matcher(graph_module.graph)
    output = next(n for n in graph_module.graph.nodes if n.op == "output")
    results = output.args[0]
    results = results if isinstance(results, (list, tuple)) else (results,)
    tensors = [r for r in results if isinstance(r, torch.fx.Node)]
    if len(tensors) != 1:
        m.refuse(f"expected one output tensor (the logits), found {len(tensors)}")
    head = m.linear(tensors[0])
    if head is None:
        m.refuse("the output is not a linear LM head", tensors[0])
    final = m.rmsnorm(head.x)
    if final is None:
        m.refuse("no final RMSNorm in front of the LM head", head.x)
    hidden, norm_kind, eps = final[0], final[3], final[2]
    activation, rope_scale, q_scale = None, 1.0, None
    inv_freq = position = None
    layers: list[LayerBinding] = []
    attention_calls: list[dict] = []
    embed = None
    while True:
        embed = m.embedding(hidden)
        if embed is not None:
            break
        if len(layers) > 512:
            m.refuse("residual chain does not end in an embedding")
        # ---- MLP half: hidden = h_mid + down(act(gate(n2)) * up(n2))
        pair = _binary(hidden, aten.add.Tensor)
        if pair is None:
            m.refuse("expected a residual add", hidden)
        mlp = None
        for skip, branch in (pair, pair[::-1]):
            down = m.linear(branch)
            gated = m.gated(down.x) if down is not None else None
            if gated is not None:
                mlp = (strip(skip), down, gated)
                break
        if mlp is None:
            m.refuse("residual branch is not down(act(gate) * up)", hidden)
        h_mid, down, (gate, up, act) = mlp
        norm2 = m.rmsnorm(gate.x)
        if norm2 is None or up.x is not gate.x or norm2[0] is not h_mid:
            m.refuse("gate and up projections must read one RMSNorm of the residual stream", gate.node)
        if activation not in (None, act) or norm2[3] != norm_kind:
            m.refuse("layers disagree on activation or norm spelling", gate.node)
        if norm2[2] != eps:
            m.refuse(f"layers disagree on the RMSNorm epsilon ({norm2[2]} vs {eps})", gate.node)
        activation = act
        # ---- attention half: h_mid = h_in + o_proj(kv_attention(rope(q), rope(k), v, state))
        pair = _binary(h_mid, aten.add.Tensor)
        if pair is None:
            m.refuse("expected a residual add around attention", h_mid)
        found = None
        for skip, branch in (pair, pair[::-1]):
            o_proj = m.linear(branch)
            call = m.kv_attention(o_proj.x) if o_proj is not None else None
            if call is None and o_proj is not None:
                call = m.prefill_attention(o_proj.x) or m.prefill_state_attention(o_proj.x)
            if call is not None:
                found = (strip(skip), o_proj, call)
                break
        if found is None:
            m.refuse("residual branch is not o_proj(megabake::kv_attention(...)) or "
                     "o_proj(megabake::attention(...))", h_mid)
        h_in, o_proj, call = found
        attention_calls.append(call)
        source = strip(call["source"])
        layer_q_scale = None
        scaled = _binary(source, aten.mul.Tensor)
        if scaled is not None and _scalar(scaled[1]) is not None and m.rope(scaled[0]) is not None:
            layer_q_scale, source = float(scaled[1]), strip(scaled[0])
        rq, rk = m.rope(source), m.rope(call["key"])
        v_proj = m.linear(call["value"])
        if rq is None or rk is None or v_proj is None:
            m.refuse("attention operands are not rope(q_proj), rope(k_proj), v_proj", o_proj.node)
        (q_proj, tc, ts), (k_proj, _, _) = rq, rk
        norm1 = m.rmsnorm(q_proj.x)
        if (norm1 is None or k_proj.x is not q_proj.x or v_proj.x is not q_proj.x
                or norm1[0] is not h_in or norm1[3] != norm_kind):
            m.refuse("q, k and v projections must read one RMSNorm of the residual stream",
                     q_proj.node)
        if tc[1] != ts[1] or tc[2:] != ts[2:]:
            m.refuse("cos and sin tables disagree", q_proj.node)
        if inv_freq not in (None, tc[2]) or position not in (None, tc[3]):
            m.refuse("layers use different rotary tables", q_proj.node)
        # "no scale" (None) is a value like any other: every layer must agree with the first seen
        if layers and q_scale != layer_q_scale:
            m.refuse("layers use different query scales", q_proj.node)
        if norm1[2] != eps:
            m.refuse(f"layers disagree on the RMSNorm epsilon ({norm1[2]} vs {eps})", q_proj.node)
        rope_scale, inv_freq, position, q_scale = tc[1], tc[2], tc[3], layer_q_scale
        if any(b is not None for b in (gate.bias, up.bias)):
            m.refuse("biased gate/up projections are not covered", gate.node)
        layers.append(LayerBinding(
            input_norm=norm1[1], q_weight=q_proj.weight, k_weight=k_proj.weight,
            v_weight=v_proj.weight, o_weight=o_proj.weight, post_norm=norm2[1],
            gate_weight=gate.weight, up_weight=up.weight, down_weight=down.weight,
            key_cache=call["key_cache"], value_cache=call["value_cache"],
            valid_length=call["valid_length"], q_bias=q_proj.bias, k_bias=k_proj.bias,
            v_bias=v_proj.bias, o_bias=o_proj.bias, down_bias=down.bias,
        ))
        hidden = h_in
    if not layers:
        m.refuse("no decoder layer found")
    stateless = ["mask" in call for call in attention_calls]
    if any(stateless) != all(stateless):
        m.refuse("layers mix megabake::attention and megabake::kv_attention")
    if all(stateless):
        if mode != "prefill":
            raise ValueError("mode='decode' graphs must update KV state through "
                             "megabake::kv_attention (megabake::attention found); use mode='prefill'")
        layers.reverse()
        return _prefill_program(m, graph_module, layers, attention_calls[::-1], embed, head, final,
                                norm_kind, eps, activation, rope_scale, q_scale, inv_freq, position)
    if mode != "decode":
        raise ValueError("mode='prefill' graphs must not update KV state "
                         "(megabake::kv_attention found); use mode='decode'")
    layers.reverse()
    first = layers[0]
    cache = _val(m.placeholders[first.key_cache])
    if cache.dim() != 4:
        m.refuse("KV caches must be [batch, capacity, kv_heads, head_dim]")
    batch, capacity, kv_heads, head_dim = cache.shape
    lengths = _val(m.placeholders[first.valid_length])
    if lengths.dtype != torch.int32 or tuple(lengths.shape) not in ((1,), (batch,)):
        m.refuse(f"valid_length must be int32 [1] (shared by the batch) or [{batch}] (one per "
                 f"row), got {lengths.dtype} {tuple(lengths.shape)}")
    length_count = int(lengths.shape[0])
    for index, layer in enumerate(layers):
        for name, position_ in (("key_cache", layer.key_cache), ("value_cache", layer.value_cache)):
            other = _val(m.placeholders[position_])
            if tuple(other.shape) != tuple(cache.shape) or other.dtype != cache.dtype:
                m.refuse(f"layer {index}: {name} is {other.dtype} {tuple(other.shape)}, layer 0's "
                         f"caches are {cache.dtype} {tuple(cache.shape)}")
        other = _val(m.placeholders[layer.valid_length])
        if other.dtype != torch.int32 or tuple(other.shape) != tuple(lengths.shape):
            m.refuse(f"layer {index}: valid_length is {other.dtype} {tuple(other.shape)}, layer 0's "
                     f"is int32 {tuple(lengths.shape)}")
    q_rows = _shape(m.placeholders[first.q_weight])[0]
    embed_weight, ids, scale_index = embed
    vocab, hidden_size = _shape(m.placeholders[head.weight])
    ids_shape = _shape(m.placeholders[ids])
    if tuple(ids_shape) != (batch, 1):
        m.refuse(f"decode takes input_ids of shape [{batch}, 1], got {ids_shape}")
    program = DecoderProgram(
        mode="decode", batch=batch, tokens=1, hidden=hidden_size, heads=q_rows // head_dim,
        kv_heads=kv_heads, head_dim=head_dim,
        intermediate=_shape(m.placeholders[first.gate_weight])[0], vocab=vocab,
        capacity=capacity, norm=norm_kind, eps=eps, activation=activation, embed_scale=None,
        rope_scale=rope_scale, q_scale=q_scale, softmax_scale=head_dim ** -0.5,
        inv_freq_dtype="bf16" if _val(m.placeholders[inv_freq]).dtype == torch.bfloat16 else "f32",
        input_ids=ids, position_ids=position, embed_weight=embed_weight, inv_freq=inv_freq,
        final_norm=final[1], lm_head_weight=head.weight, layers=tuple(layers),
        lm_head_bias=head.bias, embed_scale_arg=scale_index, length_count=length_count,
    )
    return program


def _classify_mask(m, mask, batch, tokens, node):
    """(causal?, tensor to upload or None) of an evaluated additive mask."""
    if (not isinstance(mask, torch.Tensor) or mask.dim() != 4 or mask.shape[1] != 1
            or tuple(mask.shape[2:]) != (tokens, tokens) or mask.shape[0] not in (1, batch)):
        m.refuse("the attention mask is not [1 or batch, 1, tokens, tokens]", node)
    mask = mask.to(torch.bfloat16)
    allowed = torch.tril(torch.ones(tokens, tokens, dtype=torch.bool, device=mask.device))
    floor = torch.finfo(torch.bfloat16).min
    expected = torch.where(allowed, torch.zeros((), dtype=torch.bfloat16, device=mask.device),
                           torch.full((), floor, dtype=torch.bfloat16, device=mask.device))
    causal = bool((mask == expected).all())
    return causal, (None if causal else mask.contiguous())


def _prefill_program(m, graph_module, layers, calls, embed, head, final, norm_kind, eps, activation,
                     rope_scale, q_scale, inv_freq, position) -> DecoderProgram:
    from torch.utils._python_dispatch import _disable_current_modes

    first = calls[0]
    batch, tokens, heads, head_dim = _shape(first["source"])
    kv_shape = _shape(first["key"])
    if len(kv_shape) != 4 or kv_shape[:2] != (batch, tokens) or kv_shape[3] != head_dim:
        m.refuse("megabake::attention operands must be [batch, tokens, heads, head_dim]",
                 first["node"])
    kv_heads = kv_shape[2]
    for call in calls:
        same_mask = call["mask"] is first["mask"] or (
            call["mask"] is not None and first["mask"] is not None
            and strip(call["mask"]) is strip(first["mask"]))
        same_mask = same_mask and bool(call.get("causal")) == bool(first.get("causal"))
        if (_shape(call["source"]) != (batch, tokens, heads, head_dim)
                or _shape(call["key"]) != kv_shape or _shape(call["value"]) != kv_shape
                or call["scale"] != first["scale"] or not same_mask):
            m.refuse("layers disagree on attention shapes, scale or mask", call["node"])
    embed_weight, ids, scale_index = embed
    if tuple(_shape(m.placeholders[ids])) != (batch, tokens):
        m.refuse(f"prefill takes input_ids of shape [{batch}, {tokens}]")
    # recognition runs inside the compiler's tracing modes (fake tensors): the mask constant
    # has to be computed and inspected for real
    capacity, length_count = 0, 1
    if first.get("causal"):  # the stateful prefill operator is causal by definition
        causal, mask_tensor = True, None
        cache = _val(m.placeholders[first["key_cache"]])
        if tuple(cache.shape[0:1]) != (batch,) or tuple(cache.shape[2:]) != (kv_heads, head_dim):
            m.refuse("KV caches must be [batch, capacity, kv_heads, head_dim]", first["node"])
        capacity = int(cache.shape[1])
        if capacity < tokens:
            m.refuse(f"prompt of {tokens} tokens exceeds the KV capacity {capacity}", first["node"])
        lengths = _val(m.placeholders[first["valid_length"]])
        if lengths.dtype != torch.int32 or tuple(lengths.shape) not in ((1,), (batch,)):
            m.refuse(f"valid_length must be int32 [1] or [{batch}], got {lengths.dtype} "
                     f"{tuple(lengths.shape)}", first["node"])
        length_count = int(lengths.shape[0])
    elif first["mask"] is not None:
        mask = m.constant(first["mask"], graph_module)
        with _disable_current_modes():
            causal, mask_tensor = _classify_mask(m, mask, batch, tokens, first["node"])
    else:  # no mask at all: every key visible, expressed as an all-zero additive mask
        with _disable_current_modes():
            causal, mask_tensor = False, torch.zeros(1, 1, tokens, tokens, dtype=torch.bfloat16)
    vocab, hidden_size = _shape(m.placeholders[head.weight])
    return DecoderProgram(
        mode="prefill", batch=batch, tokens=tokens, hidden=hidden_size, heads=heads,
        kv_heads=kv_heads, head_dim=head_dim,
        intermediate=_shape(m.placeholders[layers[0].gate_weight])[0], vocab=vocab,
        capacity=capacity, norm=norm_kind, eps=eps, activation=activation, embed_scale=None, rope_scale=rope_scale,
        q_scale=q_scale, softmax_scale=first["scale"],
        inv_freq_dtype="bf16" if _val(m.placeholders[inv_freq]).dtype == torch.bfloat16 else "f32",
        input_ids=ids, position_ids=position, embed_weight=embed_weight, inv_freq=inv_freq,
        final_norm=final[1], lm_head_weight=head.weight, layers=tuple(layers),
        lm_head_bias=head.bias, embed_scale_arg=scale_index, causal=causal, mask=mask_tensor,
        length_count=length_count,
    )
