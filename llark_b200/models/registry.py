"""Which model class serves a checkpoint folder, decided from its config.json.

The reference picks the class by substring of the model name (m2t/models/utils.py:126-203, mirrored by
llark_b200.models.utils.load_pretrained_model) and registers its classes with transformers' Auto* tables under
`model_type` (m2t/models/llamav2.py:422-423). Checkpoints of that kind carry `model_type`; native checkpoints carry
`architecture`. `model_class_for` covers both, `load_model` loads a native one onto the GPU."""
import json
import os

import torch

NATIVE = {}        # architecture -> (module, class name); imported on demand
HF_MODEL_TYPES = {"wrapped_llamav2": ("llark_b200.models.llamav2", "WrappedLlamav2ForCausalLM"),
                  "mpt": ("llark_b200.models.mpt", "WrappedMPTForCausalLM")}


def register_native(architecture, module, class_name):
    NATIVE[architecture] = (module, class_name)


register_native("Kelutar", "llark_b200.models.kelutar", "KelutarForCausalLM")
register_native("Golavik", "llark_b200.models.golavik", "GolavikForCausalLM")
register_native("Gubulorn", "llark_b200.models.gubulorn", "GubulornForCausalLM")
register_native("Tokatar", "llark_b200.models.tokatar", "TokatarForCausalLM")


def read_config(folder):
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
        return json.load(f)


def model_class_for(config: dict):
    import importlib

    arch = config.get("architecture")
    if arch in NATIVE:
        module, name = NATIVE[arch]
    elif config.get("model_type") in HF_MODEL_TYPES:
        module, name = HF_MODEL_TYPES[config["model_type"]]
    else:
        raise ValueError(f"no model class for architecture={arch!r} / model_type={config.get('model_type')!r}; "
                         f"known: {sorted(NATIVE)} and {sorted(HF_MODEL_TYPES)}")
    return getattr(importlib.import_module(module), name)


def load_model(folder, dtype=torch.bfloat16, device="cuda:0"):
    """The model of a native checkpoint folder (config.json + model.safetensors) on `device`."""
    config = read_config(folder)
    cls = model_class_for(config)
    if config.get("architecture") not in NATIVE:
        raise ValueError("checkpoints with `model_type` load through llark_b200.models.utils.load_pretrained_model")
    return cls.from_pretrained(folder, dtype=dtype, device=device)
