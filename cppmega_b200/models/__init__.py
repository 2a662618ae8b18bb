from .nam56r import NAM56RModel, build_model, HybridLayer, MTPLayer  # noqa: F401
