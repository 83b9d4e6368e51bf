"""gpt_neox_b200: a Blackwell-native (sm_100a) large-LM training framework with the user surface
of GPT-NeoX: NeoX YAML configs, deepy/train/generate/eval entry points, Megatron/DeepSpeed
checkpoint layout."""
__version__ = "0.1.0"
