"""Which adjoints does the running autograd pass actually need?

``ctx.needs_input_grad`` only reflects ``requires_grad`` at forward time; a ``grad`` call that
targets coordinates may prune parameter-only ancestors.  Same policy as the reference
(ictc_o3/autograd/adjoint_requirements.py:12-26): ask the engine, keep every declared gradient
when the query is unavailable.
"""
import torch


def required_gradients(inputs, declared):
    if not hasattr(torch._C, "_will_engine_execute_node") or torch._C._are_functorch_transforms_active():
        return tuple(bool(d) for d in declared)
    result = []
    for tensor, needed in zip(inputs, declared):
        if not needed:
            result.append(False)
            continue
        try:
            node = torch.autograd.graph.get_gradient_edge(tensor).node
            result.append(bool(torch._C._will_engine_execute_node(node)))
        except (RuntimeError, AttributeError, AssertionError):
            result.append(True)
    return tuple(result)
