"""Text models: tokenizer, UIE, ERNIE sequence / token classification helpers."""
from .tokenizer import Encoding, ErnieTokenizer, PyErnieTokenizer, write_synthetic_vocab  # noqa: F401
from .uie import SchemaLanguage, SchemaNode, UIEModel, UIEResult  # noqa: F401
from .ernie import ErnieSeqCls, ErnieTokenCls  # noqa: F401
from .spm_tokenizer import XLMRobertaTokenizer  # noqa: F401
