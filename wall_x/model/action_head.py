from wallx_b200.models.action_head import ActionProcessor, Normalizer, SinusoidalPosEmb  # noqa: F401
