"""Model zoo with Hugging Face parameter names, and the scheduling recipes."""
from .bert import (BertConfig, BertForMaskedLM, BertModel, RobertaForMaskedLM,  # noqa: F401
                   RobertaModel, mlm_loss, roberta_config)
