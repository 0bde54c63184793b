"""Which adjoints does the running autograd pass actually need?

``ctx.needs_input_grad`` is fixed when the forward runs: it says which inputs *could* receive a gradient.
A later ``autograd.grad`` call that asks for coordinates only prunes the branches that lead to parameters,
and skipping those adjoints saves whole kernel launches.  The autograd engine can be asked whether the
gradient edge of an input will run in the current pass; when that query does not exist (older torch, or
functorch transforms active) or fails, every declared gradient is kept.  The reference applies the same
policy (ictc_o3/autograd/adjoint_requirements.py:12-26).
"""
import torch

_QUERY = getattr(torch._C, "_will_engine_execute_node", None)


def _runs_in_this_pass(tensor) -> bool:
    try:
        edge = torch.autograd.graph.get_gradient_edge(tensor)
        return bool(_QUERY(edge.node))
    except (RuntimeError, AttributeError, AssertionError):
        return True          # not inside a backward pass, or no gradient edge: stay on the safe side


def required_gradients(inputs, declared):
    """Tuple of booleans, one per input: declared AND reached by the running backward pass."""
    flags = [bool(flag) for flag in declared]
    if _QUERY is None or torch._C._are_functorch_transforms_active():
        return tuple(flags)
    return tuple(flag and _runs_in_this_pass(t) for t, flag in zip(inputs, flags))
