"""pyre_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

    from pyre_b200 import Engine, SamplingParams
    engine = Engine("path/to/model", dtype="bfloat16")
    outs = engine.generate([[1, 2, 3]], SamplingParams(max_new_tokens=8))
"""

from .config import EngineConfig, ModelConfig, Qwen2Config, load_config, register_architecture
from .sampling import SamplingParams

__version__ = "0.1.0"

__all__ = ["Engine", "EngineConfig", "ModelConfig", "Qwen2Config", "RequestOutput", "SamplingParams",
           "load_config", "load_model", "register_architecture"]


def __getattr__(name):
    # the engine pulls in torch.cuda and the kernel loader; import it on first use
    if name in ("Engine", "RequestOutput"):
        from .engine import engine as _engine
        return getattr(_engine, name)
    if name == "load_model":
        from .models.model import load_model
        return load_model
    raise AttributeError(name)
