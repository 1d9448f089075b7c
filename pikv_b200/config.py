"""Model configuration dict with the keys of core/single/config.py:4-17 (read at construction time)."""
import torch

config = {
    "num_experts": 4,
    "hidden_size": 256,
    "num_heads": 8,
    "kv_cache_size": 128,
    "epochs": 10,
    "batch_size": 32,
    "learning_rate": 1e-3,
    "device": torch.device("cuda" if torch.cuda.is_available() else "cpu"),
    "pyramidal_cache": True,
    "cache_decrement": 10,
    "num_layers": 5,
    "vocab_size": 50257,
}
