"""The Qwen3 dense decoder: its name in config.json and the names of its tensors.

Tensor names are the ones tools/export.py:90-99 lists.
"""
from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from .layout import ModelLayout
from .model import expected_tensors


class Qwen3Architecture:
    name = "Qwen3ForCausalLM"

    def parse_config(self, raw):
        return Qwen3Config.from_dict(raw)

    def layout(self, spec):
        layers = []
        for l in range(len(spec.layers)):
            p = f"model.layers.{l}."
            names = {
                ("mixer_norm", "weight"): p + "input_layernorm.weight",
                ("mixer", "wq"): p + "self_attn.q_proj.weight",
                ("mixer", "wk"): p + "self_attn.k_proj.weight",
                ("mixer", "wv"): p + "self_attn.v_proj.weight",
                ("mixer", "wo"): p + "self_attn.o_proj.weight",
                ("mixer", "q_norm"): p + "self_attn.q_norm.weight",
                ("mixer", "k_norm"): p + "self_attn.k_norm.weight",
                ("ffn_norm", "weight"): p + "post_attention_layernorm.weight",
                ("ffn", "gate"): p + "mlp.gate_proj.weight",
                ("ffn", "up"): p + "mlp.up_proj.weight",
                ("ffn", "down"): p + "mlp.down_proj.weight",
            }
            layers.append(names)
        return ModelLayout(embed="model.embed_tokens.weight", final_norm="model.norm.weight", head="lm_head.weight",
                           layers=layers)

    def info(self, spec):
        """The model's name and sizes as abacus's --info prints them (src/main.c:143-145)."""
        m, f = spec.layers[0].mixer, spec.layers[0].ffn
        return (f"qwen3 dim={spec.hidden} hidden={f.inter} layers={len(spec.layers)} heads={m.n_heads}/{m.n_kv_heads} "
                f"head_dim={m.head_dim} vocab={spec.vocab}")

    def tensor_names(self, spec, available=None):
        return expected_tensors(spec, self.layout(spec), available)


register_architecture(Qwen3Architecture())
