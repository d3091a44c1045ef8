from .base import ByteTokenizer, Tokenizer
from .hf import HFTokenizer
from .llama3 import Llama3Tokenizer
from .sentencepiece import SentencePieceTokenizer
