from . import qwen3  # registers Qwen3ForCausalLM
