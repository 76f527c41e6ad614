"""Model zoo with Hugging Face parameter names, and the scheduling recipes."""
from .bert import (BertConfig, BertForMaskedLM, BertModel, RobertaForMaskedLM,  # noqa: F401
                   RobertaModel, mlm_loss, roberta_config)
from .gpt import (Conv1D, GPT2LMHeadModel, GPTConfig, GPTNeoForCausalLM,  # noqa: F401,E402
                  causal_lm_loss)
from .opt import OPTConfig, OPTForCausalLM, OPTModel  # noqa: F401,E402
from .t5 import T5Config, T5ForConditionalGeneration, seq2seq_loss  # noqa: F401,E402
from .albert import AlbertConfig, AlbertForMaskedLM, AlbertModel  # noqa: F401,E402
from .wideresnet import (WideResNet, WideResNetWithLoss, get_wideresnet,  # noqa: F401,E402
                         wideresnet_config)
