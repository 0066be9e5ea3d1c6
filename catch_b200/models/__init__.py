"""Model definitions used by the examples, tests and benchmarks."""
from .bert import BertConfig, BertForSequenceClassification  # noqa: F401
from .resnet import resnet18, resnet50, resnet101  # noqa: F401
