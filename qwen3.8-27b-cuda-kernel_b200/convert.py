"""Checkpoint -> .q38 converter with the quantiser and the packer running on the GPU.

    python qwen3.8-27b-cuda-kernel_b200/convert.py --model <hf dir> --out model.q38 [--recipe default] [--layers N]
                                                   [--device cuda]

Front end of the same conversion the reference's tools/convert.py performs (plan and tensor semantics:
tools/convert.py:214-339; config mapping: tools/convert.py:103-152): reads `config.json` and the `*.safetensors`
shards of a Hugging Face checkpoint directory, de-interleaves q / gate, folds the (1 + w) RMSNorm weights into the
following projection, interleaves gate / up rows, and writes the `.q38` file. Quantisation (`bqformat.quantize_matrix`,
the 48-candidate squared-error search) and bit-plane packing are tensor arithmetic and run on `--device`; on a GPU
they produce the bytes of the CPU run, which the golden fixtures pin to the reference's own output. `--layers N`
keeps the first N layers (the reference's option for truncated test models). No tokenizer resources are embedded.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _package():
    name = "q38b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, HERE / "__init__.py", submodule_search_locations=[str(HERE)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def text_config(model_dir: Path) -> dict:
    """The header `config` block from a Hugging Face config.json (text part of a multimodal config if present)."""
    raw = json.loads((model_dir / "config.json").read_text())
    tc = raw.get("text_config", raw)
    rope = tc.get("rope_parameters") or tc.get("rope_scaling") or {}
    if rope.get("rope_type", rope.get("type", "default")) != "default":
        raise ValueError("only unscaled RoPE is supported")
    if tc.get("hidden_act", "silu") != "silu" or tc.get("attention_bias", False):
        raise ValueError("unsupported activation or attention bias")
    layers = tc["num_hidden_layers"]
    kinds = tc.get("layer_types") or ["full_attention" if (i + 1) % tc.get("full_attention_interval", 4) == 0
                                      else "linear_attention" for i in range(layers)]
    eos = []
    gen = model_dir / "generation_config.json"
    if gen.exists():
        e = json.loads(gen.read_text()).get("eos_token_id", [])
        eos = e if isinstance(e, list) else [e]
    if not eos:
        e = tc.get("eos_token_id", [])
        eos = e if isinstance(e, list) else [e]
    head_dim = tc["head_dim"]
    partial = rope.get("partial_rotary_factor", tc.get("partial_rotary_factor", 0.25))
    return {
        "architecture": "qwen3_5_dense", "hidden_size": tc["hidden_size"], "num_layers": layers, "layer_types": list(kinds),
        "vocab_size": tc["vocab_size"], "intermediate_size": tc["intermediate_size"],
        "num_attention_heads": tc["num_attention_heads"], "num_key_value_heads": tc["num_key_value_heads"],
        "head_dim": head_dim, "rotary_dim": int(head_dim * partial),
        "rope_theta": float(rope.get("rope_theta", tc.get("rope_theta", 10_000_000))),
        "linear_num_key_heads": tc["linear_num_key_heads"], "linear_num_value_heads": tc["linear_num_value_heads"],
        "linear_key_head_dim": tc["linear_key_head_dim"], "linear_value_head_dim": tc["linear_value_head_dim"],
        "linear_conv_kernel_dim": tc["linear_conv_kernel_dim"], "rms_norm_eps": float(tc.get("rms_norm_eps", 1e-6)),
        "max_position_embeddings": tc["max_position_embeddings"],
        "tie_word_embeddings": bool(raw.get("tie_word_embeddings", tc.get("tie_word_embeddings", False))),
        "norm_folded": True, "eos_token_ids": eos,
    }


class SafetensorsSource:
    """Tensors of a checkpoint directory by their Hugging Face names without the model prefix
    (`layers.3.mlp.up_proj.weight`, `embed_tokens.weight`, `norm.weight`, `lm_head.weight`), read lazily."""

    PREFIXES = ("", "model.", "model.language_model.", "language_model.model.", "language_model.")

    def __init__(self, model_dir: Path):
        from safetensors import safe_open
        self._open = safe_open
        self.where: dict[str, Path] = {}
        index = model_dir / "model.safetensors.index.json"
        if index.exists():
            for name, shard in json.loads(index.read_text())["weight_map"].items():
                self.where[name] = model_dir / shard
        else:
            for shard in sorted(model_dir.glob("*.safetensors")):
                with safe_open(str(shard), framework="pt") as f:
                    for name in f.keys():
                        self.where[name] = shard
        if not self.where:
            raise FileNotFoundError(f"no safetensors shards in {model_dir}")

    def __contains__(self, name: str) -> bool:
        return any(p + name in self.where for p in self.PREFIXES)

    def __getitem__(self, name: str):
        for p in self.PREFIXES:
            full = p + name
            if full in self.where:
                with self._open(str(self.where[full]), framework="pt") as f:
                    return f.get_tensor(full)
        raise KeyError(name)


def convert(model_dir: Path, out: Path, recipe: str = "default", layers: int | None = None, device: str = "cuda",
            grid: int = 24) -> dict:
    _package()
    from q38b200 import synth
    cfg = text_config(model_dir)
    if layers is not None and layers < cfg["num_layers"]:
        cfg["num_layers"] = layers
        cfg["layer_types"] = cfg["layer_types"][:layers]
    src = SafetensorsSource(model_dir)
    if cfg["tie_word_embeddings"] and "lm_head.weight" not in src:
        class Tied:
            def __getitem__(self, name):
                return src["embed_tokens.weight" if name == "lm_head.weight" else name]
        source = Tied()
    else:
        source = src
    synth.write_q38(out, cfg, source, recipe=recipe, grid=grid, device=device)
    return cfg


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="Hugging Face checkpoint directory (config.json + *.safetensors)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--recipe", default="default")
    ap.add_argument("--layers", type=int, default=None, help="keep only the first N layers")
    ap.add_argument("--device", default="cuda", help="where the quantiser and the packer run (cuda or cpu)")
    ap.add_argument("--grid", type=int, default=24, help="stretch factors per range end of the scale search")
    a = ap.parse_args(argv)
    cfg = convert(Path(a.model), Path(a.out), a.recipe, a.layers, a.device, a.grid)
    print(f"wrote {a.out}: {cfg['num_layers']} layers, hidden {cfg['hidden_size']}, vocab {cfg['vocab_size']}, recipe {a.recipe}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
