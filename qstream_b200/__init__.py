"""qstream_b200: a small model library with generation of its own for one NVIDIA B200.

From a model folder (config.json + safetensors) or seeded random weights to generated
tokens: typed configuration and architecture registry, weights by tensor name, layers
put together from parts, a paged per-sequence cache, one batched step function, a
generation loop, sampling, and hand-written sm_100a kernels under it all.

    import qstream_b200 as qs
    model = qs.load_model("folder", dtype="bfloat16")
    engine = qs.Engine(model, qs.EngineConfig(max_batch=8))
    out = qs.generate(engine, [[1, 2, 3], [4, 5]], max_new_tokens=16,
                      sampling=qs.SamplingConfig.greedy())
"""
from .errors import QsError, QStreamError, error_string
from .config import GptjConfig, config_from_dict, load_config, register_architecture
from .weights import InitScales, write_model_folder
from .sampling import SamplingConfig
from .engine import CausalLM, Engine, EngineConfig, GenerationResult, Generator, load_model


def generate(engine, prompts, max_new_tokens=256, sampling=None, stop_tokens=None, callback=None,
             emit_stop_token=False) -> GenerationResult:
    """Generate for a list of token-id prompts; see `Generator.generate`."""
    return Generator(engine).generate(prompts, max_new_tokens, sampling, stop_tokens, callback,
                                      emit_stop_token)


__version__ = "0.1.0"
__all__ = ["QsError", "QStreamError", "error_string", "GptjConfig", "config_from_dict", "load_config",
           "register_architecture", "InitScales", "write_model_folder", "SamplingConfig", "CausalLM",
           "Engine", "EngineConfig", "GenerationResult", "Generator", "load_model", "generate"]
