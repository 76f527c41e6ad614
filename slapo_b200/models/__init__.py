"""Model zoo with Hugging Face parameter names, and the scheduling recipes."""
from .bert import (BertConfig, BertForMaskedLM, BertModel, RobertaForMaskedLM,  # noqa: F401
                   RobertaModel, mlm_loss, roberta_config)
from .gpt import (Conv1D, GPT2LMHeadModel, GPTConfig, GPTNeoForCausalLM,  # noqa: F401,E402
                  causal_lm_loss)
from .opt import OPTConfig, OPTForCausalLM, OPTModel  # noqa: F401,E402
