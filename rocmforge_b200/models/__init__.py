from . import qwen2      # registers "Qwen2ForCausalLM"
from . import rifizen    # registers "Rifizen"
from . import vilulorn   # registers "Vilulorn"
from . import figalix    # registers "Figalix"
