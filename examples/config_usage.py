#!/usr/bin/env python
"""Configuration values, builder, store, per-plugin settings and layering of file, environment
and command line (counterpart of examples/config_usage.rs plus the layering the reference lists
as future work)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from coeus_b200.prelude import ConfigBuilder, ConfigStore, PluginConfigManager


def main(argv=()) -> dict:
    cfg = (ConfigBuilder.map().with_("name", "example").with_("max_length", 512)
           .with_("lowercase", True).with_("dropout", 0.1).build())
    m = cfg.as_map()
    print("builder:", {k: str(v) for k, v in m.items()})
    store = ConfigStore.new()
    store.set("model.hidden_dim", 1024)
    store.set("model.num_layers", 16)
    store.set("tokenizer.type", "bpe")
    overrides = ConfigStore.new()
    overrides.set("model.num_layers", 24)
    store.merge(overrides)
    store.load_mapping({"train": {"lr": 3e-4, "steps": 100}})
    store.load_env(environ={"COEUS_TRAIN__LR": "1e-4"})
    rest = store.load_args(["--train.steps=200", *argv])
    pm = PluginConfigManager.new()
    pm.set_plugin_key("bpe_tokenizer", "vocab_size", 50000)
    return {"layers": store.get("model.num_layers").as_integer(),
            "lr": store.get("train.lr").as_float(), "steps": store.get("train.steps").as_integer(),
            "vocab": pm.get_plugin_key("bpe_tokenizer", "vocab_size").as_integer(),
            "name": m["name"].as_string(), "rest": rest}


if __name__ == "__main__":
    print(main(sys.argv[1:]))
