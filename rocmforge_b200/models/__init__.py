from . import qwen2      # registers "Qwen2ForCausalLM"
