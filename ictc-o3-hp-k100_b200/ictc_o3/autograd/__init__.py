from .adjoint_requirements import required_gradients  # noqa: F401
