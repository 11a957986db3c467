"""Layers, initialisers and losses."""
from .init import Init, initialize  # noqa: F401
from .layers import (ELU, GELU, LSTM, RNN, AdaptiveAvgPool2d, AvgPool2d, BatchNorm2d, Buffer, ComputeStats, Conv1d,  # noqa: F401
                     Conv2d, ConvTranspose2d, Dropout, Embedding, Flatten, GELUTanh, LayerNorm, Linear, LSTMCell, MaxPool2d, Mish, Param,
                     ReLU, RMSNorm, RNNCell, Sequential, Sigmoid, Softmax, Swish, Tanh, manual_seed, seq)
from .loss import (CrossEntropyLoss, MSELoss, bce_loss, bce_with_logits_loss, cross_entropy_loss, huber_loss,  # noqa: F401
                   kl_div_loss, l1_loss, mse_loss, nll_loss)
