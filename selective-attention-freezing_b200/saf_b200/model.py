"""Prefill of the whole model around the blocks: token embedding, the transformer blocks, final LayerNorm and the
last-position language-model head, as GPT.forward does for inference (nanogpt/model.py:1326-1337, 1373-1416;
`logits = lm_head(x[:, -1:, :])`).  Same module names as the reference (`transformer.wte`, `transformer.h`,
`transformer.ln_f`, `lm_head`, tied embedding) so its checkpoints load.  RoPE positions only."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .attention import rope_tables
from .block import LayerNorm, SafBlock


class SafGPT(nn.Module):
    def __init__(self, config):
        super().__init__()
        assert getattr(config, "position_encoding", "rope") == "rope", "only RoPE positions are implemented"
        self.config = config
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd),
            h=nn.ModuleList([SafBlock(config, layer_idx=i) for i in range(config.n_layer)]),
            ln_f=LayerNorm(config.n_embd, bias=getattr(config, "bias", False)),
        ))
        self.lm_head = nn.Linear(config.n_embd, config.vocab_size, bias=False)
        self.transformer.wte.weight = self.lm_head.weight   # weight tying (nanogpt/model.py:1337)
        self._rope = None

    def rope(self, T, device):
        if self._rope is None or self._rope[0].shape[2] != T or self._rope[0].device != device:
            hd = self.config.n_embd // self.config.n_head
            cos, sin = rope_tables(hd, T, base=getattr(self.config, "rope_base", 10000.0), device=device)
            self._rope = (cos.view(1, 1, T, hd), sin.view(1, 1, T, hd))
        return self._rope

    def forward_hidden(self, idx):
        x = self.transformer.wte(idx)
        rope = self.rope(idx.shape[1], idx.device)
        for block in self.transformer.h:
            x = block(x, rope=rope)
        return self.transformer.ln_f(x)

    def forward(self, idx, targets=None):
        """GPT.forward of the reference (nanogpt/model.py:1401-1417): with targets, logits at every position and
        the mean cross-entropy (ignore_index -1); without, next-token logits at the last position, (B, 1, vocab),
        and None."""
        x = self.forward_hidden(idx)
        if targets is not None:
            logits = self.lm_head(x)
            loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1), ignore_index=-1)
            return logits, loss
        return F.linear(x[:, -1:, :], self.lm_head.weight), None
