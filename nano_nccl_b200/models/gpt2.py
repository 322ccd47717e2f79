"""GPT-2-small layer stack: the list of parameter shapes (124M elements: hidden 768, 12 layers,
vocabulary 50257, context 1024) used as the gradient list of the bucketed all-reduce benchmark, and
a tiny trainable module of the same structure for data-parallel smoke tests."""
import torch


def gpt2_small_shapes(hidden=768, layers=12, vocab=50257, context=1024):
    shapes = [(vocab, hidden), (context, hidden)]
    for _ in range(layers):
        shapes += [(hidden,), (hidden,),                       # ln_1
                   (hidden, 3 * hidden), (3 * hidden,),        # attn.c_attn
                   (hidden, hidden), (hidden,),                # attn.c_proj
                   (hidden,), (hidden,),                       # ln_2
                   (hidden, 4 * hidden), (4 * hidden,),        # mlp.c_fc
                   (4 * hidden, hidden), (hidden,)]            # mlp.c_proj
    shapes += [(hidden,), (hidden,)]                           # ln_f
    return shapes


class _Block(torch.nn.Module):
    def __init__(self, hidden, heads):
        super().__init__()
        self.ln_1 = torch.nn.LayerNorm(hidden)
        self.attn = torch.nn.MultiheadAttention(hidden, heads, batch_first=True)
        self.ln_2 = torch.nn.LayerNorm(hidden)
        self.mlp = torch.nn.Sequential(torch.nn.Linear(hidden, 4 * hidden), torch.nn.GELU(), torch.nn.Linear(4 * hidden, hidden))

    def forward(self, x):
        h = self.ln_1(x)
        x = x + self.attn(h, h, h, need_weights=False)[0]
        return x + self.mlp(self.ln_2(x))


class TinyGPT2(torch.nn.Module):
    def __init__(self, vocab=512, context=64, hidden=64, layers=2, heads=4):
        super().__init__()
        self.wte = torch.nn.Embedding(vocab, hidden)
        self.wpe = torch.nn.Embedding(context, hidden)
        self.blocks = torch.nn.ModuleList([_Block(hidden, heads) for _ in range(layers)])
        self.ln_f = torch.nn.LayerNorm(hidden)

    def forward(self, tokens):
        pos = torch.arange(tokens.shape[1], device=tokens.device)
        x = self.wte(tokens) + self.wpe(pos)
        for b in self.blocks:
            x = b(x)
        return self.ln_f(x) @ self.wte.weight.t()
