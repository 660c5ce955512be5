"""Text models (reference: text/): WordPiece tokenizer and BERT encoder with heads."""
from .wordpiece import WordPiece
from .bert import Bert, BertConfig, BertForMaskedLM, BertForSequenceClassification
