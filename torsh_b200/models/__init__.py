"""Model zoo."""
from .gpt2 import GPT2Config, GPT2LMHeadModel, GPT2Model, GPTForCausalLM

__all__ = ["GPT2Config", "GPT2Model", "GPTForCausalLM", "GPT2LMHeadModel"]
