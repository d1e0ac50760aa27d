"""Public engine classes, same names as the reference's ``llm.py``."""
from .engine.llm_engine.predictor_llm_engine import PredictorLLMEngine
from .engine.llm_engine.talker_llm_engine import TalkerLLMEngine


class TalkerLLM(TalkerLLMEngine):
    pass


class PredictorLLM(PredictorLLMEngine):
    pass


def LLM(model: str, **kwargs):
    """The engine registered for the architecture that ``model``'s config.json names (``models/registry.py``)."""
    import json
    import os
    from .models.registry import resolve
    with open(os.path.join(model, "config.json")) as f:
        arch = resolve(json.load(f))
    return arch.engine_cls(model, **kwargs)
