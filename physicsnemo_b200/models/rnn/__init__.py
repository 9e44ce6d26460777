from .rnn import One2ManyRNN, Seq2SeqRNN
