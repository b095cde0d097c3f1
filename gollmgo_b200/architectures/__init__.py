from . import llama     # registers "LlamaForCausalLM"
from . import tekenex   # registers "Tekenex"
