"""Building blocks of the GNMT translation stages, as plain torch modules.

The reference's stage files for translation (runtime/translation/models/gnmt_large/gpus=4/stage*.py)
are made of `torch.nn` layers plus four custom blocks from runtime/translation/seq2seq/models/
(`EmuBidirLSTM`, encoder.py:25-64; `BahdanauAttention`, attention.py:12-170; `RecurrentAttention`,
decoder.py:13-62; `Classifier`, decoder.py:65-95) and the `LabelSmoothing` criterion
(seq2seq/train/smoothing.py:7-34).  Those files are not available where this library runs, so the
blocks are restated here with the same parameter names, shapes, construction order (hence the same
initial values under a fixed seed) and arithmetic.  They are user-level modules: StageRuntime swaps
their LSTM / Linear / Embedding leaves for native ones (layers.nativize) like any other stage.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def _revert_varlen_torch(x, lengths):
    """out[t,b] = x[len[b]-1-t, b] for t < len[b], else 0 (pure torch; differentiable)."""
    T, B = x.shape[0], x.shape[1]
    t = torch.arange(T, device=x.device).unsqueeze(1)                       # [T,1]
    L = lengths.to(x.device).unsqueeze(0)                                    # [1,B]
    src = (L - 1 - t).clamp(min=0)                                           # [T,B]
    valid = (t < L)
    idx = src.view(T, B, *([1] * (x.dim() - 2))).expand_as(x)
    out = torch.gather(x, 0, idx)
    return out * valid.view(T, B, *([1] * (x.dim() - 2))).to(x.dtype)


class EmuBidirLSTM(nn.Module):
    """A bidirectional LSTM layer emulated by two one-direction LSTMs that share the parameters of a
    (never executed) bidirectional nn.LSTM; the backward direction runs on the per-sequence
    time-reversed input and its output is reversed back."""

    def __init__(self, input_size, hidden_size):
        super().__init__()
        self.bidir = nn.LSTM(input_size, hidden_size, 1, True, False, bidirectional=True)
        self.layer1 = nn.LSTM(input_size, hidden_size, 1, True, False)
        self.layer2 = nn.LSTM(input_size, hidden_size, 1, True, False)
        for name in ("weight_ih_l0", "weight_hh_l0", "bias_ih_l0", "bias_hh_l0"):
            setattr(self.layer1, name, getattr(self.bidir, name))
            setattr(self.layer2, name, getattr(self.bidir, name + "_reverse"))

    def forward(self, input, lengths):
        return emu_bidir_reference(self, input, lengths)


def emu_bidir_reference(emu, input, lengths):
    lengths = lengths.cpu().long()
    T = input.shape[0]
    mask = (torch.arange(T).unsqueeze(1) < lengths.unsqueeze(0)).unsqueeze(-1).to(input.device).type_as(input)
    rev = _revert_varlen_torch(input, lengths)
    out_rev = _revert_varlen_torch(emu.layer2(rev)[0], lengths)
    out_fwd = emu.layer1(input)[0] * mask
    return torch.cat([out_fwd, out_rev], dim=2)


class BahdanauAttention(nn.Module):
    """Normalised additive attention: score(q,k) = v . tanh(Wq q + Wk k + b), v = g * a / |a|."""

    def __init__(self, query_size, key_size, num_units, normalize=True, dropout=0, batch_first=False):
        super().__init__()
        self.normalize = normalize
        self.batch_first = batch_first
        self.num_units = num_units
        self.linear_q = nn.Linear(query_size, num_units, bias=False)
        self.linear_k = nn.Linear(key_size, num_units, bias=False)
        self.linear_att = nn.Parameter(torch.Tensor(num_units))
        self.dropout = nn.Dropout(dropout)
        self.register_buffer('mask', None)
        if normalize:
            self.normalize_scalar = nn.Parameter(torch.Tensor(1))
            self.normalize_bias = nn.Parameter(torch.Tensor(num_units))
        else:
            self.register_parameter('normalize_scalar', None)
            self.register_parameter('normalize_bias', None)
        stdv = 1. / math.sqrt(num_units)
        self.linear_att.data.uniform_(-stdv, stdv)
        if normalize:
            self.normalize_scalar.data.fill_(stdv)
            self.normalize_bias.data.zero_()

    def set_mask(self, context_len, context):
        max_len = context.size(1) if self.batch_first else context.size(0)
        steps = torch.arange(0, max_len, dtype=torch.int64, device=context.device)
        self.mask = steps >= context_len.unsqueeze(1)

    def calc_score(self, q, k):
        b, t_k, n = k.size()
        t_q = q.size(1)
        s = q.unsqueeze(2).expand(b, t_q, t_k, n) + k.unsqueeze(1).expand(b, t_q, t_k, n)
        if self.normalize:
            s = s + self.normalize_bias
            a = self.linear_att.to(torch.float32)
            v = (a / a.norm()).to(self.normalize_scalar) * self.normalize_scalar
        else:
            v = self.linear_att
        return torch.tanh(s).matmul(v)

    def forward(self, query, keys):
        if not self.batch_first:
            keys = keys.transpose(0, 1)
            if query.dim() == 3:
                query = query.transpose(0, 1)
        single = query.dim() == 2
        if single:
            query = query.unsqueeze(1)
        b, t_k, t_q = query.size(0), keys.size(1), query.size(1)
        scores = self.calc_score(self.linear_q(query), self.linear_k(keys))
        if self.mask is not None:
            scores.data.masked_fill_(self.mask.unsqueeze(1).expand(b, t_q, t_k), -65504.0)
        probs = self.dropout(F.softmax(scores, dim=-1))
        context = torch.bmm(probs, keys)
        if single:
            return context.squeeze(1), probs.squeeze(1)
        if not self.batch_first:
            return context.transpose(0, 1), probs.transpose(0, 1)
        return context, probs


class RecurrentAttention(nn.Module):
    """LSTM layer followed by attention over the encoder output."""

    def __init__(self, input_size, context_size, hidden_size, num_layers=1, bias=True, batch_first=False, dropout=0):
        super().__init__()
        self.rnn = nn.LSTM(input_size, hidden_size, num_layers, bias, batch_first)
        self.attn = BahdanauAttention(hidden_size, context_size, context_size, normalize=True, batch_first=batch_first)
        self.dropout = nn.Dropout(dropout)

    def forward(self, inputs, hidden, context, context_len):
        self.attn.set_mask(context_len, context)
        rnn_outputs, hidden = self.rnn(inputs, hidden)
        attn_outputs, scores = self.attn(rnn_outputs, context)
        return self.dropout(rnn_outputs), hidden, attn_outputs, scores


class Classifier(nn.Module):
    def __init__(self, in_features, out_features):
        super().__init__()
        self.out_features = out_features
        self.classifier = nn.Linear(in_features, out_features)

    def forward(self, x):
        return self.classifier(x)[..., :self.out_features]


class LabelSmoothing(nn.Module):
    """NLL with label smoothing over [T,B,V] logits; PAD targets are skipped; sum divided by B."""

    def __init__(self, padding_idx, smoothing=0.0):
        super().__init__()
        self.padding_idx = padding_idx
        self.confidence = 1.0 - smoothing
        self.smoothing = smoothing

    def forward(self, output, target):
        x = output.view(output.size(0) * output.size(1), -1)
        logp = F.log_softmax(x, dim=-1, dtype=torch.float32)
        keep = target != self.padding_idx
        nll = -logp.gather(dim=-1, index=target.unsqueeze(1)).squeeze(1)[keep]
        smooth = -logp.mean(dim=-1)[keep]
        return (self.confidence * nll + self.smoothing * smooth).sum() / output.size(1)


# --------------------------------------------------------------------------- #
# the four stages of the 8+8-layer model (partitioning "gpus=4")
# --------------------------------------------------------------------------- #
class GnmtStage0(nn.Module):
    """Embedding, bidirectional layer, LSTM(2H->H), then three residual LSTM layers of the encoder."""

    def __init__(self, hidden=1024, vocab=32320, p=0.2):
        super().__init__()
        self.layer6 = nn.Embedding(vocab, hidden, padding_idx=0)
        self.layer7 = EmuBidirLSTM(hidden, hidden)
        self.layer8 = nn.Dropout(p=p)
        self.layer9 = nn.LSTM(2 * hidden, hidden)
        self.layer11 = nn.Dropout(p=p)
        self.layer12 = nn.LSTM(hidden, hidden)
        self.layer15 = nn.Dropout(p=p)
        self.layer16 = nn.LSTM(hidden, hidden)
        self.layer19 = nn.Dropout(p=p)
        self.layer20 = nn.LSTM(hidden, hidden)

    def forward(self, input0, input1):
        src, src_len = input0.clone(), input1.clone()
        x = self.layer9(self.layer8(self.layer7(self.layer6(src), src_len)))[0]
        x = self.layer12(self.layer11(x))[0] + x
        x = self.layer16(self.layer15(x))[0] + x
        return x, self.layer20(self.layer19(x))[0]


class GnmtStage1(nn.Module):
    """Last three residual encoder layers, decoder embedding, attention layer, first decoder LSTM."""

    def __init__(self, hidden=1024, vocab=32320, p=0.2):
        super().__init__()
        self.layer10 = nn.Embedding(vocab, hidden, padding_idx=0)
        self.layer12 = nn.Dropout(p=p)
        self.layer13 = nn.LSTM(hidden, hidden)
        self.layer16 = nn.Dropout(p=p)
        self.layer17 = nn.LSTM(hidden, hidden)
        self.layer20 = nn.Dropout(p=p)
        self.layer21 = nn.LSTM(hidden, hidden)
        self.layer24 = RecurrentAttention(hidden, hidden, hidden)
        self.layer27 = nn.Dropout(p=p)
        self.layer29 = nn.LSTM(2 * hidden, hidden)

    def forward(self, input1, input2, input0, input3):
        # input1: residual stream of the encoder, input0: output of its last LSTM so far,
        # input2: source lengths, input3: decoder input tokens
        x = input0.clone() + input1.clone()
        src_len, tgt = input2.clone(), input3.clone()
        emb = self.layer10(tgt)
        x = self.layer13(self.layer12(x))[0] + x
        x = self.layer17(self.layer16(x))[0] + x
        x = self.layer21(self.layer20(x))[0] + x
        rnn_out, _, attn, _ = self.layer24(emb, None, x, src_len)
        y = self.layer29(torch.cat([self.layer27(rnn_out), attn], 2), None)[0]
        return attn, y


class GnmtStage2(nn.Module):
    """Four residual decoder layers, each fed with [dropout(x), attention]."""

    def __init__(self, hidden=1024, p=0.2):
        super().__init__()
        self.layer9 = nn.Dropout(p=p)
        self.layer11 = nn.LSTM(2 * hidden, hidden)
        self.layer14 = nn.Dropout(p=p)
        self.layer16 = nn.LSTM(2 * hidden, hidden)
        self.layer19 = nn.Dropout(p=p)
        self.layer21 = nn.LSTM(2 * hidden, hidden)
        self.layer24 = nn.Dropout(p=p)
        self.layer26 = nn.LSTM(2 * hidden, hidden)
        self.layer29 = nn.Dropout(p=p)

    def forward(self, input8, input0):
        x, attn = input0.clone(), input8.clone()
        for drop, lstm in ((self.layer9, self.layer11), (self.layer14, self.layer16), (self.layer19, self.layer21),
                           (self.layer24, self.layer26)):
            x = lstm(torch.cat([drop(x), attn], 2), None)[0] + x
        return x, torch.cat([self.layer29(x), attn], 2), attn


class GnmtStage3(nn.Module):
    """Last two decoder layers and the vocabulary classifier."""

    def __init__(self, hidden=1024, vocab=32320, p=0.2):
        super().__init__()
        self.layer5 = nn.LSTM(2 * hidden, hidden)
        self.layer8 = nn.Dropout(p=p)
        self.layer10 = nn.LSTM(2 * hidden, hidden)
        self.layer13 = Classifier(hidden, vocab)

    def forward(self, input3, input2, input0):
        # input0: [dropout(x), attention] from the previous stage, input2: x, input3: attention
        cat_in, x, attn = input0.clone(), input2.clone(), input3.clone()
        x = self.layer5(cat_in, None)[0] + x
        x = self.layer10(torch.cat([self.layer8(x), attn], 2), None)[0] + x
        return self.layer13(x)
