from . import llama     # registers "LlamaForCausalLM"
