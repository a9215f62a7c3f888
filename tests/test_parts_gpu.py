"""Each part of a layer alone against the plain implementation, and the generality of the
composition: a toy architecture, defined here, with a mixer that keeps per-request state of its
own, a layer that runs twice and a layer that reads another layer's cache, is registered, built
from a model folder and stepped through the engine's step function without any change to the
package's files."""
import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping

import numpy as np
import pytest
import torch

import plain_model
import tiny_configs
from helpers import random_prompts, read_tensors, write_model

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------------------------
# Parts alone
# ----------------------------------------------------------------------------------------------
def one_layer_runner(folder, dtype, page):
    from velox_b200.cache.manager import CacheManager
    from velox_b200.engine.engine import load_model
    from velox_b200.engine.runner import ModelRunner

    _, spec, model = load_model(folder, dtype, torch.device("cuda:0"), max_position=256)
    cache = CacheManager(model.cache_groups, num_pages=40, page_size=page, max_model_len=256, max_num_seqs=4)
    return spec, model, cache, ModelRunner(model, cache, max_num_seqs=4, max_num_batched_tokens=256)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case,page", [("tiny_a", 4), ("tiny_c", 16)])
def test_parts_of_one_layer(tmp_path, dtype, case, page):
    from velox_b200.engine.runner import StepChunk
    from velox_b200.parts.base import HiddenState

    cfg = tiny_configs.ALL[case]
    write_model(str(tmp_path), cfg, seed=3, dtype="bfloat16")
    tensors = {k: v.double() for k, v in read_tensors(str(tmp_path)).items()}
    spec, model, cache, runner = one_layer_runner(str(tmp_path), dtype, page)
    tol = 2e-5 if dtype == torch.float32 else 3e-2

    T = 37
    tokens = random_prompts(cfg["vocab_size"], (T,), seed=1)[0]
    seq = cache.new_sequence("s")
    assert cache.acquire_slot(seq) and cache.append_slots(seq, T)
    ctx, ids, rows, _ = runner.prepare([StepChunk(seq, tokens, ())])
    block = model.blocks[0]
    E = cfg["hidden_size"]
    heads, kv_heads = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim") or E // heads
    eps = cfg["rms_norm_eps"]
    p = "model.layers.0."

    def close(got, want, what):
        got, want = got.double().cpu(), want.double()
        err = (got - want).abs().max().item()
        assert err <= tol * max(want.abs().max().item(), 1e-3), f"{what}: {err:.3e}"

    # embedding
    resid = torch.zeros(256, E, device="cuda")
    model.embedding.forward(ids, resid, ctx)
    h0 = tensors["model.embed_tokens.weight"][torch.tensor(tokens)]
    close(resid[:T], h0, "embedding")

    # norm (no pending delta)
    normed = torch.zeros(256, E, dtype=dtype, device="cuda")
    block.norm_mixer.forward(resid, None, normed, T)
    x0 = plain_model.rms_norm(h0, tensors[p + "input_layernorm.weight"], eps)
    close(normed[:T], x0, "norm")

    # mixer: attention over the cache, whole prompt
    angles = plain_model.rope_angles(D, cfg["rope_theta"], 1.0, torch.arange(T))
    want_attn = plain_model.attention_block(x0, tensors, p + "self_attn.", heads, kv_heads, D,
                                            angles.cos().double(), angles.sin().double(), None)
    exact_in = x0.to(dtype).cuda()
    padded = torch.zeros(256, E, dtype=dtype, device="cuda")
    padded[:T] = exact_in
    mixed = block.mixer.forward(padded, ctx, runner.layer_caches[0])
    close(mixed[:T], want_attn, "attention mixer")

    # feed-forward
    y = torch.randn(T, E, generator=torch.Generator().manual_seed(2)).double()
    padded[:T] = y.to(dtype).cuda()
    ff = block.feed_forward.forward(padded, ctx)
    want_ff = plain_model.swiglu_mlp(y.to(dtype).double(), tensors[p + "mlp.gate_proj.weight"],
                                     tensors[p + "mlp.up_proj.weight"], tensors[p + "mlp.down_proj.weight"])
    close(ff[:T], want_ff, "feed-forward")

    # block: norm + mixer + norm + feed-forward around the residual stream
    seq2 = cache.new_sequence("s2")
    assert cache.acquire_slot(seq2) and cache.append_slots(seq2, T)
    ctx2, ids2, _, _ = runner.prepare([StepChunk(seq2, tokens, ())])
    resid2 = torch.zeros(256, E, device="cuda")
    model.embedding.forward(ids2, resid2, ctx2)
    hidden = HiddenState(resid=resid2, delta=None)
    block.forward(hidden, ctx2, runner.layer_caches[0])
    torch.cuda.synchronize()
    want_h = plain_model.decoder_layer(h0, tensors, 0, cfg, angles.cos().double(), angles.sin().double(), None)
    pending = 0 if hidden.delta is None else hidden.delta[:T].float()
    close(hidden.resid[:T] + pending, want_h, "block")

    # lm head on selected rows
    final = torch.zeros(8, E, dtype=dtype, device="cuda")
    z = torch.randn(3, E, generator=torch.Generator().manual_seed(4))
    final[:3] = z.to(dtype).cuda()
    logits = model.lm_head.forward(final, 3, ctx2)
    head = tensors["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else tensors["lm_head.weight"]
    close(logits, z.to(dtype).double() @ head.T, "lm head")
    runner.check_status()


# ----------------------------------------------------------------------------------------------
# A toy architecture defined in this file
# ----------------------------------------------------------------------------------------------
TOY_ARCH = "ToyStateForCausalLM"


def register_toy():
    from velox_b200.config import ModelConfig, register_architecture
    from velox_b200.parts import Mixer, StateSpec, register_part
    from velox_b200.parts.base import CacheNeeds
    from velox_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

    @register_part("mixer", "toy_running_mean")
    class RunningMean(Mixer):
        """out[t] = W @ mean(x[0..t]): the mean is carried in per-request state (sum and count),
        so a portion continues where the previous one stopped.  Written with torch ops: it is a
        test double, not a product kernel."""

        def __init__(self, params, weights, dtype, device):
            super().__init__(params, weights, dtype, device)
            self.size = int(params["hidden_size"])
            self.w = self.expect("proj.weight", (self.size, self.size))

        def cache_needs(self):
            return CacheNeeds(state=StateSpec(shape=(self.size + 1,), dtype=torch.float32))

        def forward(self, x, ctx, cache):
            out = ctx.workspace.get("toy.out", (ctx.workspace.max_tokens, self.size), self.dtype)
            slots = ctx.seq_slots.tolist()
            starts = ctx.q_start.tolist()
            for s, (n, slot) in enumerate(zip(ctx.q_lens_host, slots)):
                rows = x[starts[s] : starts[s] + n].float()
                state = cache.state[slot]
                sums = state[: self.size] + rows.cumsum(0)
                counts = state[self.size] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                mean = sums / counts.unsqueeze(1)
                out[starts[s] : starts[s] + n] = (mean @ self.w.float().T).to(self.dtype)
                state[: self.size] = sums[-1]
                state[self.size] = counts[-1]
            return out

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        num_attention_heads: int = 2
        head_dim: int = 16
        intermediate_size: int = 64

        def to_json_dict(self):
            return {
                "architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "num_hidden_layers": self.num_hidden_layers, "max_position_embeddings": self.max_position_embeddings,
                "tie_word_embeddings": self.tie_word_embeddings, "num_attention_heads": self.num_attention_heads,
                "head_dim": self.head_dim, "intermediate_size": self.intermediate_size,
            }

    def parse(cfg: Mapping[str, Any]) -> ToyConfig:
        return ToyConfig(
            architecture=TOY_ARCH, vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
            num_hidden_layers=cfg["num_hidden_layers"], max_position_embeddings=cfg["max_position_embeddings"],
            tie_word_embeddings=cfg["tie_word_embeddings"], num_attention_heads=cfg["num_attention_heads"],
            head_dim=cfg["head_dim"], intermediate_size=cfg["intermediate_size"],
        )

    def build(c: ToyConfig) -> ModelSpec:
        E, H, D, I, V = c.hidden_size, c.num_attention_heads, c.head_dim, c.intermediate_size, c.vocab_size
        mat = lambda *src: WeightSpec(tuple(src), "matrix")
        vec = lambda *src: WeightSpec(tuple(src), "vector")
        rms = lambda name: PartSpec("rms", {"size": E, "eps": 1e-5},
                                    {"weight": vec(TensorSource(name, (E,), "one_plus_normal"))})
        position = PartSpec("rotary_half", {"head_dim": D, "rotary_dim": D // 2, "theta": 500.0,
                                            "scaling_factor": 1.0, "max_position": c.max_position_embeddings})

        def ffn(p):
            return PartSpec("swiglu", {"hidden_size": E, "intermediate_size": I}, {
                "gate_up.weight": mat(TensorSource(p + "gate.weight", (I, E)), TensorSource(p + "up.weight", (I, E))),
                "down.weight": mat(TensorSource(p + "down.weight", (E, I)))})

        def attn(p):
            return PartSpec("attention", {"hidden_size": E, "num_heads": H, "num_kv_heads": H, "head_dim": D,
                                          "qkv_bias": False, "window": None, "softmax_scale": 1 / math.sqrt(D)}, {
                "qkv.weight": mat(TensorSource(p + "q.weight", (H * D, E)), TensorSource(p + "k.weight", (H * D, E)),
                                  TensorSource(p + "v.weight", (H * D, E))),
                "out.weight": mat(TensorSource(p + "o.weight", (E, H * D)))})

        layers = [
            LayerSpec("pre_norm", attn("l0.attn."), ffn("l0.ffn."),
                      {"mixer": rms("l0.n1"), "feed_forward": rms("l0.n2")}, position),
            LayerSpec("pre_norm", PartSpec("toy_running_mean", {"hidden_size": E},
                                           {"proj.weight": mat(TensorSource("l1.mix.weight", (E, E)))}),
                      ffn("l1.ffn."), {"mixer": rms("l1.n1"), "feed_forward": rms("l1.n2")}, None),
            LayerSpec("pre_norm", attn("l2.attn."), ffn("l2.ffn."),
                      {"mixer": rms("l2.n1"), "feed_forward": rms("l2.n2")}, position),
        ]
        embed = TensorSource("embed.weight", (V, E))
        return ModelSpec(
            architecture=TOY_ARCH, hidden_size=E, vocab_size=V, max_position=c.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": E}, {"weight": mat(embed)}),
            layers=tuple(layers),
            # layer 0, the stateful layer, layer 0 again (its own cache), layer 2 reading the
            # cache of the first entry, the stateful layer again (its own state)
            schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, cache_of=0), ScheduleEntry(1)),
            final_norm=rms("final.weight"),
            lm_head=PartSpec("linear_head", {"hidden_size": E, "vocab_size": V}, {"weight": mat(embed)}),
        )

    register_architecture(TOY_ARCH, parse, build)


def toy_plain_logits(tensors, cfg, tokens):
    """Plain float64 forward of the toy model, whole sequence."""
    t = {k: v.double() for k, v in tensors.items()}
    E, H, D = cfg["hidden_size"], cfg["num_attention_heads"], cfg["head_dim"]
    T = len(tokens)
    h = t["embed.weight"][torch.tensor(tokens)]
    rot = D // 2
    ang = plain_model.rope_angles(rot, 500.0, 1.0, torch.arange(T)).double()

    def rope(x):
        return torch.cat([plain_model.rotate_half(x[..., :rot], ang.cos(), ang.sin()), x[..., rot:]], -1)

    def attn(x, p, shared_kv=None):
        q = rope((x @ t[p + "q.weight"].T).view(T, H, D))
        if shared_kv is None:
            k = rope((x @ t[p + "k.weight"].T).view(T, H, D))
            v = (x @ t[p + "v.weight"].T).view(T, H, D)
        else:
            k, v = shared_kv
        o = plain_model.causal_attention(q, k, v, 1 / math.sqrt(D))
        return o.reshape(T, H * D) @ t[p + "o.weight"].T, (k, v)

    def ffn(x, p):
        return plain_model.swiglu_mlp(x, t[p + "gate.weight"], t[p + "up.weight"], t[p + "down.weight"])

    def running_mean(x):
        mean = x.cumsum(0) / torch.arange(1, T + 1, dtype=torch.float64).unsqueeze(1)
        return mean @ t["l1.mix.weight"].T

    norm = lambda x, name: plain_model.rms_norm(x, t[name], 1e-5)
    kv_first = None
    for entry, (layer, shared) in enumerate([(0, False), (1, False), (0, False), (2, True), (1, False)]):
        p = f"l{layer}."
        x = norm(h, p + "n1")
        if layer == 1:
            mixed = running_mean(x)
        else:
            mixed, kv = attn(x, p + "attn.", kv_first if shared else None)
            if entry == 0:
                kv_first = kv
        h = h + mixed
        h = h + ffn(norm(h, p + "n2"), p + "ffn.")
    return norm(h, "final.weight") @ t["embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_stateful_mixer(tmp_path, dtype):
    from velox_b200.config import unregister_architecture
    from velox_b200.engine.replay import TraceReplayer
    from velox_b200.parts import unregister_part
    from velox_b200.weights import write_random_model

    register_toy()
    try:
        cfg = {"architectures": [TOY_ARCH], "vocab_size": 97, "hidden_size": 48, "num_hidden_layers": 3,
               "max_position_embeddings": 128, "tie_word_embeddings": True, "num_attention_heads": 2,
               "head_dim": 16, "intermediate_size": 72}
        folder = str(tmp_path)
        write_random_model(folder, cfg, seed=5, dtype="bfloat16", std=0.08)
        tensors = read_tensors(folder)
        prompts = random_prompts(97, (50, 23), seed=3)
        want = [toy_plain_logits(tensors, cfg, p) for p in prompts]
        replayer = TraceReplayer(folder, dtype, max_tokens=128, block_size=8)
        a, b = prompts
        # a: 20 tokens, then 2, then one by one beside b's portions; b ends, its slot is reused by c = a again
        got_a = np.zeros((50, 97), np.float32)
        got_b = np.zeros((23, 97), np.float32)
        plan = [
            [("a", 0, 20)], [("a", 20, 2), ("b", 0, 9)], [("a", 22, 1), ("b", 9, 13)], [("b", 22, 1), ("a", 23, 1)],
            [("a", 24, 26)],
        ]
        for step, entries in enumerate(plan):
            rec = {"step": step, "end": [],
                   "entries": [{"id": n, "tokens": (a if n == "a" else b)[s : s + c], "want": list(range(c))} for n, s, c in entries]}
            if step == 3:
                rec["end"] = ["b"]
            out = replayer.run_step(rec)
            row = 0
            for n, s, c in entries:
                (got_a if n == "a" else got_b)[s : s + c] = out[row : row + c]
                row += c
        # a new request in b's old slot must start from zero state
        out_c = replayer.run_step({"step": 9, "entries": [{"id": "c", "tokens": b, "want": list(range(23))}], "end": ["c", "a"]})
        tol = 2e-5 if dtype == "float32" else 3e-2
        for got, ref, what in ((got_a, want[0], "a"), (got_b, want[1], "b"), (out_c, want[1], "c")):
            err = (torch.from_numpy(got).double() - ref).abs().max().item()
            assert err <= tol * ref.abs().max().item(), (what, err, ref.abs().max().item())
        assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    finally:
        unregister_architecture(TOY_ARCH)
        unregister_part("mixer", "toy_running_mean")


# ----------------------------------------------------------------------------------------------
# A second toy architecture: a feed-forward that routes, and a position encoding of its own
# ----------------------------------------------------------------------------------------------
ROUTED_ARCH = "ToyRoutedForCausalLM"
ROUTER_SCALE = 40.0  # router logits far enough apart that no token sits between two experts


def register_routed_toy():
    from velox_b200.config import ModelConfig, register_architecture
    from velox_b200.parts import register_part
    from velox_b200.parts.base import FeedForward, PositionEncoding
    from velox_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(FeedForward):
        """out[t] = p * W2[e] relu(W1[e] x[t]) for the expert e with the largest router logit,
        p its softmax probability (float32 router).  Torch ops: a test double."""

        def __init__(self, params, weights, dtype, device):
            super().__init__(params, weights, dtype, device)
            self.E, self.I, self.N = int(params["hidden_size"]), int(params["inner"]), int(params["experts"])
            self.scale = float(params["router_scale"])
            self.router = self.expect("router.weight", (self.N, self.E))
            self.w1 = self.expect("w1", (self.N * self.I, self.E))
            self.w2 = self.expect("w2", (self.N * self.E, self.I))

        def forward(self, x, ctx):
            T = ctx.num_tokens
            out = ctx.workspace.get("toy.routed", (ctx.workspace.max_tokens, self.E), self.dtype)
            rows = x[:T].float()
            probs = torch.softmax(self.scale * (rows @ self.router.float().T), dim=-1)
            weight, expert = probs.max(dim=-1)
            result = torch.zeros(T, self.E, device=x.device, dtype=torch.float32)
            for e in range(self.N):
                mine = (expert == e).nonzero().flatten()
                if mine.numel() == 0:
                    continue
                w1 = self.w1[e * self.I : (e + 1) * self.I].float()
                w2 = self.w2[e * self.E : (e + 1) * self.E].float()
                result[mine] = (torch.relu(rows[mine] @ w1.T) @ w2.T) * weight[mine].unsqueeze(1)
            out[:T] = result.to(self.dtype)
            return out

    @register_part("position", "toy_rotary_pairs")
    class RotaryPairs(PositionEncoding):
        """Rotation of neighbouring pairs (2i, 2i + 1) of every head by position * theta^(-i/(D/2)),
        and the write of k and v into the paged cache, with torch ops."""

        def __init__(self, params, weights, dtype, device):
            super().__init__(params, weights, dtype, device)
            self.D = int(params["head_dim"])
            self.inv_freq = (float(params["theta"]) ** (-torch.arange(self.D // 2, dtype=torch.float32) / (self.D // 2))).to(device)

        def rotate_and_store(self, qkv, ctx, slots, k_cache, v_cache, num_heads, num_kv_heads):
            T, D = ctx.num_tokens, self.D
            ang = ctx.positions[:T].float().unsqueeze(1) * self.inv_freq
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

            def rotate(x):  # [T, heads, D]
                even, odd = x[..., 0::2].float(), x[..., 1::2].float()
                return torch.stack([even * cos - odd * sin, even * sin + odd * cos], dim=-1).flatten(-2).to(x.dtype)

            q = qkv[:T, : num_heads * D].view(T, num_heads, D)
            k = qkv[:T, num_heads * D : (num_heads + num_kv_heads) * D].view(T, num_kv_heads, D)
            v = qkv[:T, (num_heads + num_kv_heads) * D :].view(T, num_kv_heads, D)
            q.copy_(rotate(q))
            if k_cache is not None:
                keep = (slots[:T] >= 0).nonzero().flatten()
                where = slots[:T][keep].long()
                k_cache.view(-1, num_kv_heads, D)[where] = rotate(k)[keep]
                v_cache.view(-1, num_kv_heads, D)[where] = v[keep]

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        num_attention_heads: int = 3
        num_key_value_heads: int = 1
        head_dim: int = 32
        inner: int = 40
        experts: int = 3

        def to_json_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "num_hidden_layers": self.num_hidden_layers, "max_position_embeddings": self.max_position_embeddings,
                    "tie_word_embeddings": self.tie_word_embeddings, "num_attention_heads": self.num_attention_heads,
                    "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim, "inner": self.inner,
                    "experts": self.experts}

    def parse(cfg: Mapping[str, Any]) -> RoutedConfig:
        keys = ("vocab_size", "hidden_size", "num_hidden_layers", "max_position_embeddings", "tie_word_embeddings",
                "num_attention_heads", "num_key_value_heads", "head_dim", "inner", "experts")
        return RoutedConfig(architecture=ROUTED_ARCH, **{k: cfg[k] for k in keys})

    def build(c: RoutedConfig) -> ModelSpec:
        E, H, G, D, V = c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.vocab_size
        mat = lambda *src: WeightSpec(tuple(src), "matrix")
        vec = lambda *src: WeightSpec(tuple(src), "vector")
        rms = lambda name: PartSpec("rms", {"size": E, "eps": 1e-5},
                                    {"weight": vec(TensorSource(name, (E,), "one_plus_normal"))})
        position = PartSpec("toy_rotary_pairs", {"head_dim": D, "theta": 200.0})
        layers = []
        for i in range(c.num_hidden_layers):
            p = f"l{i}."
            attn = PartSpec("attention", {"hidden_size": E, "num_heads": H, "num_kv_heads": G, "head_dim": D,
                                          "qkv_bias": False, "window": None, "softmax_scale": 1 / math.sqrt(D)}, {
                "qkv.weight": mat(TensorSource(p + "q.weight", (H * D, E)), TensorSource(p + "k.weight", (G * D, E)),
                                  TensorSource(p + "v.weight", (G * D, E))),
                "out.weight": mat(TensorSource(p + "o.weight", (E, H * D)))})
            ffn = PartSpec("toy_top1_experts", {"hidden_size": E, "inner": c.inner, "experts": c.experts,
                                                "router_scale": ROUTER_SCALE}, {
                "router.weight": vec(TensorSource(p + "router.weight", (c.experts, E))),
                "w1": mat(TensorSource(p + "w1", (c.experts * c.inner, E))),
                "w2": mat(TensorSource(p + "w2", (c.experts * E, c.inner)))})
            layers.append(LayerSpec("pre_norm", attn, ffn, {"mixer": rms(p + "n1"), "feed_forward": rms(p + "n2")}, position))
        embed = TensorSource("embed.weight", (V, E))
        return ModelSpec(
            architecture=ROUTED_ARCH, hidden_size=E, vocab_size=V, max_position=c.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": E}, {"weight": mat(embed)}),
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(c.num_hidden_layers)),
            final_norm=rms("final.weight"),
            lm_head=PartSpec("linear_head", {"hidden_size": E, "vocab_size": V}, {"weight": mat(embed)}),
        )

    register_architecture(ROUTED_ARCH, parse, build)


def routed_plain_logits(tensors, cfg, tokens):
    """Plain float64 forward of the routed toy model, whole sequence; also the smallest gap
    between the two largest router probabilities (a tie there is a coin toss for any engine)."""
    t = {k: v.double() for k, v in tensors.items()}
    E, H, G, D = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    I, N, T = cfg["inner"], cfg["experts"], len(tokens)
    h = t["embed.weight"][torch.tensor(tokens)]
    inv_freq = 200.0 ** (-torch.arange(D // 2, dtype=torch.float64) / (D // 2))
    ang = torch.arange(T, dtype=torch.float64).unsqueeze(1) * inv_freq
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rotate(x):
        even, odd = x[..., 0::2], x[..., 1::2]
        return torch.stack([even * cos - odd * sin, even * sin + odd * cos], dim=-1).flatten(-2)

    norm = lambda x, name: plain_model.rms_norm(x, t[name], 1e-5)
    margin = float("inf")
    for i in range(cfg["num_hidden_layers"]):
        p = f"l{i}."
        x = norm(h, p + "n1")
        q = rotate((x @ t[p + "q.weight"].T).view(T, H, D))
        k = rotate((x @ t[p + "k.weight"].T).view(T, G, D)).repeat_interleave(H // G, dim=1)
        v = (x @ t[p + "v.weight"].T).view(T, G, D).repeat_interleave(H // G, dim=1)
        o = plain_model.causal_attention(q, k, v, 1 / math.sqrt(D))
        h = h + o.reshape(T, H * D) @ t[p + "o.weight"].T
        x = norm(h, p + "n2")
        probs = torch.softmax(ROUTER_SCALE * (x @ t[p + "router.weight"].T), dim=-1)
        top2 = probs.topk(2, dim=-1).values
        margin = min(margin, float((top2[:, 0] - top2[:, 1]).min()))
        weight, expert = probs.max(dim=-1)
        out = torch.zeros(T, E, dtype=torch.float64)
        for e in range(N):
            mine = (expert == e).nonzero().flatten()
            w1, w2 = t[p + "w1"][e * I : (e + 1) * I], t[p + "w2"][e * E : (e + 1) * E]
            out[mine] = (torch.relu(x[mine] @ w1.T) @ w2.T) * weight[mine].unsqueeze(1)
        h = h + out
    return norm(h, "final.weight") @ t["embed.weight"].T, margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_routed_feed_forward_and_its_own_position_encoding(tmp_path, dtype):
    """A feed-forward that routes tokens to experts and a position encoding that rotates pairs,
    both defined here, in a model built, loaded and stepped by the framework as it is."""
    from velox_b200.config import unregister_architecture
    from velox_b200.engine.replay import TraceReplayer
    from velox_b200.parts import unregister_part
    from velox_b200.weights import write_random_model

    register_routed_toy()
    try:
        cfg = {"architectures": [ROUTED_ARCH], "vocab_size": 61, "hidden_size": 56, "num_hidden_layers": 2,
               "max_position_embeddings": 96, "tie_word_embeddings": True, "num_attention_heads": 3,
               "num_key_value_heads": 1, "head_dim": 32, "inner": 40, "experts": 3}
        folder = str(tmp_path)
        write_random_model(folder, cfg, seed=15, dtype="bfloat16", std=0.1)
        tensors = read_tensors(folder)
        prompts = random_prompts(61, (40, 17), seed=8)
        refs = [routed_plain_logits(tensors, cfg, p) for p in prompts]
        assert min(m for _, m in refs) > 0.05, "pick another seed: two experts nearly tie for a token"
        replayer = TraceReplayer(folder, dtype, max_tokens=128, block_size=8)
        a, b = prompts
        got_a, got_b = np.zeros((40, 61), np.float32), np.zeros((17, 61), np.float32)
        plan = [[("a", 0, 30)], [("a", 30, 1), ("b", 0, 15)], [("a", 31, 1), ("b", 15, 1)], [("a", 32, 8), ("b", 16, 1)]]
        for step, entries in enumerate(plan):
            rec = {"step": step, "end": ["a", "b"] if step == len(plan) - 1 else [],
                   "entries": [{"id": n, "tokens": (a if n == "a" else b)[s : s + c], "want": list(range(c))} for n, s, c in entries]}
            out = replayer.run_step(rec)
            row = 0
            for n, s, c in entries:
                (got_a if n == "a" else got_b)[s : s + c] = out[row : row + c]
                row += c
        tol = 2e-5 if dtype == "float32" else 3e-2
        for got, (ref, _), what in ((got_a, refs[0], "a"), (got_b, refs[1], "b")):
            err = (torch.from_numpy(got).double() - ref).abs().max().item()
            assert err <= tol * ref.abs().max().item(), (what, err, ref.abs().max().item())
        assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    finally:
        unregister_architecture(ROUTED_ARCH)
        unregister_part("feed_forward", "toy_top1_experts")
        unregister_part("position", "toy_rotary_pairs")


# ----------------------------------------------------------------------------------------------
# A third toy architecture: attention layers of different head sizes in one model
# ----------------------------------------------------------------------------------------------
TWO_SIZES_ARCH = "ToyTwoHeadSizesForCausalLM"
TWO_SIZES_LAYERS = ((4, 2, 16), (2, 1, 32), (4, 4, 16))  # (heads, KV heads, head size) per layer


def register_two_head_sizes():
    from velox_b200.config import ModelConfig, register_architecture
    from velox_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

    @dataclass(frozen=True)
    class Config(ModelConfig):
        intermediate_size: int = 64

        def to_json_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "num_hidden_layers": self.num_hidden_layers, "max_position_embeddings": self.max_position_embeddings,
                    "tie_word_embeddings": self.tie_word_embeddings, "intermediate_size": self.intermediate_size}

    def parse(cfg: Mapping[str, Any]) -> Config:
        return Config(architecture=TWO_SIZES_ARCH, vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
                      num_hidden_layers=cfg["num_hidden_layers"], max_position_embeddings=cfg["max_position_embeddings"],
                      tie_word_embeddings=cfg["tie_word_embeddings"], intermediate_size=cfg["intermediate_size"])

    def build(c: Config) -> ModelSpec:
        E, I, V = c.hidden_size, c.intermediate_size, c.vocab_size
        mat = lambda *src: WeightSpec(tuple(src), "matrix")
        vec = lambda *src: WeightSpec(tuple(src), "vector")
        rms = lambda name: PartSpec("rms", {"size": E, "eps": 1e-6}, {"weight": vec(TensorSource(name, (E,), "one_plus_normal"))})
        layers = []
        for index, (H, G, D) in enumerate(TWO_SIZES_LAYERS):
            p = f"l{index}."
            position = PartSpec("rotary_half", {"head_dim": D, "rotary_dim": D, "theta": 10000.0, "scaling_factor": 1.0,
                                                "max_position": c.max_position_embeddings})
            mixer = PartSpec("attention", {"hidden_size": E, "num_heads": H, "num_kv_heads": G, "head_dim": D, "qkv_bias": False,
                                           "window": None, "softmax_scale": 1 / math.sqrt(D)}, {
                "qkv.weight": mat(TensorSource(p + "q.weight", (H * D, E)), TensorSource(p + "k.weight", (G * D, E)),
                                  TensorSource(p + "v.weight", (G * D, E))),
                "out.weight": mat(TensorSource(p + "o.weight", (E, H * D)))})
            ffn = PartSpec("swiglu", {"hidden_size": E, "intermediate_size": I}, {
                "gate_up.weight": mat(TensorSource(p + "gate.weight", (I, E)), TensorSource(p + "up.weight", (I, E))),
                "down.weight": mat(TensorSource(p + "down.weight", (E, I)))})
            layers.append(LayerSpec("pre_norm", mixer, ffn, {"mixer": rms(p + "n1"), "feed_forward": rms(p + "n2")}, position))
        embed = TensorSource("embed.weight", (V, E))
        return ModelSpec(
            architecture=TWO_SIZES_ARCH, hidden_size=E, vocab_size=V, max_position=c.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": E}, {"weight": mat(embed)}),
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            final_norm=rms("final.weight"),
            lm_head=PartSpec("linear_head", {"hidden_size": E, "vocab_size": V}, {"weight": mat(embed)}))

    register_architecture(TWO_SIZES_ARCH, parse, build)


def two_sizes_plain_logits(tensors, tokens):
    t = {k: v.double() for k, v in tensors.items()}
    T = len(tokens)
    h = t["embed.weight"][torch.tensor(tokens)]
    for index, (H, G, D) in enumerate(TWO_SIZES_LAYERS):
        p = f"l{index}."
        ang = plain_model.rope_angles(D, 10000.0, 1.0, torch.arange(T)).double()
        x = plain_model.rms_norm(h, t[p + "n1"], 1e-6)
        q = plain_model.rotate_half((x @ t[p + "q.weight"].T).view(T, H, D), ang.cos(), ang.sin())
        k = plain_model.rotate_half((x @ t[p + "k.weight"].T).view(T, G, D), ang.cos(), ang.sin())
        v = (x @ t[p + "v.weight"].T).view(T, G, D)
        o = plain_model.causal_attention(q, k, v, 1 / math.sqrt(D))
        h = h + o.reshape(T, H * D) @ t[p + "o.weight"].T
        x = plain_model.rms_norm(h, t[p + "n2"], 1e-6)
        h = h + plain_model.swiglu_mlp(x, t[p + "gate.weight"], t[p + "up.weight"], t[p + "down.weight"])
    return plain_model.rms_norm(h, t["final.weight"], 1e-6) @ t["embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_two_head_sizes(tmp_path, dtype):
    """Layers whose attention differs in head size (and in head counts) in one model: every
    signature gets a work layout and scratch of its own head size, and long single-token steps
    with split key ranges (forced here) stay right in both."""
    from velox_b200.config import unregister_architecture
    from velox_b200.engine.replay import TraceReplayer
    from velox_b200.weights import write_random_model

    register_two_head_sizes()
    try:
        cfg = {"architectures": [TWO_SIZES_ARCH], "vocab_size": 211, "hidden_size": 64, "num_hidden_layers": 3,
               "max_position_embeddings": 512, "tie_word_embeddings": True, "intermediate_size": 96}
        folder = str(tmp_path)
        write_random_model(folder, cfg, seed=8, dtype="bfloat16", std=0.08)
        tensors = read_tensors(folder)
        tokens = random_prompts(211, (300,), seed=6)[0]
        want = two_sizes_plain_logits(tensors, tokens)
        replayer = TraceReplayer(folder, dtype, max_tokens=320, block_size=16,
                                 plan_overrides={"min_split_keys": 64, "target_ctas": 4096})
        signatures = replayer.runner._signatures
        assert sorted({sig[3] for _, sig in signatures}) == [16, 32] and len(signatures) == 3
        rows, start = [], 0
        for step, n in enumerate([150, 2, 100] + [1] * 48):
            out = replayer.run_step({"step": step, "end": ["r"] if start + n == 300 else [],
                                     "entries": [{"id": "r", "tokens": tokens[start : start + n], "want": list(range(n))}]})
            rows.append(out)
            start += n
        got = torch.from_numpy(np.concatenate(rows)).double()
        tol = 2e-5 if dtype == "float32" else 3e-2
        err = (got - want).abs().max().item()
        assert err <= tol * want.abs().max().item(), (err, want.abs().max().item())
        assert replayer.cache.num_free_pages() == replayer.cache.num_total_pages
    finally:
        unregister_architecture(TWO_SIZES_ARCH)
