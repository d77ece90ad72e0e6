from .decoder import DecoderModel, expected_tensors

__all__ = ["DecoderModel", "expected_tensors", "load_model"]


def load_model(path: str, dtype, device="cuda"):
    """Reads a model folder (config.json picks the architecture) and returns (config, model)."""
    from ..config import load_config
    from ..parts import Runtime
    from ..weights import read_model_folder
    cfg = load_config(path)
    model = DecoderModel(cfg.model_spec(), read_model_folder(path), Runtime(device, dtype), where=path)
    return cfg, model
