"""Model and synthetic-input factories keyed by the model name prefix
(reference: mist/model_provider.py:53-117)."""
from __future__ import annotations

from .bert import BertModel, bert_inputs_provider
from .gpt import FalconModel, GPTModel, LLamaModel, gpt_inputs_provider
from .t5 import T5Model, t5_inputs_provider

_MODELS = {"gpt": GPTModel, "llama": LLamaModel, "falcon": FalconModel, "bert": BertModel, "t5": T5Model}
_INPUTS = {"gpt": gpt_inputs_provider, "llama": gpt_inputs_provider, "falcon": gpt_inputs_provider,
           "bert": bert_inputs_provider, "t5": t5_inputs_provider}


def family_of(name: str) -> str:
    name = name.lower()
    for fam in _MODELS:
        if name.startswith(fam):
            return fam
    raise ValueError(f"unknown model family for '{name}' (known: {sorted(_MODELS)})")


def base_model_provider(model_config, model_name=None, process_groups=None, pre_post_process_group=None,
                        pre_process=True, post_process=True, layer_range=None, sequence_parallel=False,
                        device=None, dtype=None):
    fam = family_of(model_name or model_config.name)
    return _MODELS[fam](model_config, pre_process=pre_process, post_process=post_process,
                        process_groups=process_groups, pre_post_process_group=pre_post_process_group,
                        layer_range=layer_range, sequence_parallel=sequence_parallel, device=device, dtype=dtype)


def get_inputs_provider(model_name: str):
    return _INPUTS[family_of(model_name)]
