"""The whole decode model sharded over the GPUs of one node (config 4): experts split expert-parallel
(experts / world per GPU), attention, norms, router, shared expert, embedding and lm_head replicated.

One process per GPU.  Every rank runs the same token through the same replicated attention block, routes it
(the router is replicated, so all ranks agree on the 8 experts without talking), computes the selected experts
it owns, and one all-reduce per MoE layer sums the weighted expert outputs (14 KB at batch 1).  This is the
per-token body of the reference's generate() (src/kimi_exec.cu:801-884) with its expert loop (:843-871)
spread over the ranks; the rounding points are kept: bf16(sum_k w_k * bf16(y_k)), then + bf16(shared), rounded
(:868-871, :684), the sum over slots being taken in fp32 across ranks instead of in slot order.

The kernels are the library's (MLA block, router, grouped expert GEMM, fused add + norm, lm_head); this file is
the host loop around them.  With use_graph=True the loop is captured, after a warm-up step, into one CUDA graph per
rank (the NCCL all-reduce included); it is off by default: the capture has only been exercised on two GPUs.
"""
import torch
import torch.distributed as dist

from . import lib, synth


class ExpertParallelModel:
    """provider(layer, name) -> CUDA tensor of that model tensor on this rank's device; layer -1 holds
    "embed_tokens", "norm", "lm_head".  Expert arrays ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s") come
    back already cut to this rank's experts [experts / world, ...]; everything else is the full tensor."""

    def __init__(self, cfg, provider, group=None, max_ctx=1024, use_graph=False):
        self.cfg, self.group = cfg, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        c = cfg
        if c.experts % self.world:
            raise ValueError("experts (%d) must divide over %d ranks" % (c.experts, self.world))
        self.per = c.experts // self.world
        self.base = self.rank * self.per
        self.device = provider(-1, "norm").device
        self.embed, self.norm, self.lm_head = provider(-1, "embed_tokens"), provider(-1, "norm"), provider(-1, "lm_head")
        lat_w = c.kv_rank + c.qk_rope
        self.layers = []
        for l in range(c.layers):
            L = dict(ln0=provider(l, "input_layernorm"), ln1=provider(l, "post_attention_layernorm"))
            aw = {k: provider(l, n) for k, n in (("q_a", "q_a_proj"), ("q_a_ln", "q_a_layernorm"), ("q_b", "q_b_proj"),
                                                ("kv_a", "kv_a_proj_with_mqa"), ("kv_a_ln", "kv_a_layernorm"),
                                                ("kv_b", "kv_b_proj"), ("o", "o_proj"))}
            L["mla"] = lib.MlaLayer(aw, yarn_factor=c.yarn_factor, rope_theta=c.rope_theta, rms_eps=c.rms_eps, max_batch=1,
                                    max_ctx=max_ctx, heads=c.heads, qk_nope=c.qk_nope, qk_rope=c.qk_rope, v_head=c.v_head)
            L["cache"] = torch.zeros((1, max_ctx, lat_w), dtype=torch.bfloat16, device=self.device)
            if l < c.first_dense:
                L["dense"] = tuple(provider(l, n) for n in ("gate_proj", "up_proj", "down_proj"))
            else:
                w = dict(router_w=provider(l, "router"), router_bias=provider(l, "router_bias"))
                for n in ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s"):
                    w[n] = provider(l, n)
                if c.shared_inter:
                    for n in ("shared_gate", "shared_up", "shared_down"):
                        w[n] = provider(l, n)
                L["moe"] = lib.MoeLayer(w, topk=c.topk, routed_scale=c.routed_scale, expert_base=self.base, max_tokens=2)
            self.layers.append(L)
        self.pos = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.ids_in = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.ids_out = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.zero8 = torch.zeros(c.topk, dtype=torch.int32, device=self.device)
        self.use_graph, self.graph, self.steps = use_graph, None, 0

    # ---- one token through every layer: reads self.ids_in, writes self.ids_out, advances self.pos ----
    def _body(self):
        c = self.cfg
        x = self.embed[self.ids_in.long()].contiguous()                          # [1, H]   (:802)
        n = lib.rmsnorm(x, self.layers[0]["ln0"], eps=c.rms_eps)
        for l, L in enumerate(self.layers):
            t = L["mla"].decode(n, L["cache"], self.pos)                         # :812-826
            n = lib.add_rmsnorm(x, t, L["ln1"], eps=c.rms_eps)                   # :827, :829
            if "dense" in L:
                t = lib.bf16_mlp(L["dense"][0], L["dense"][1], L["dense"][2], n)  # :831-834
            else:
                m = L["moe"]
                ids, wts = lib.router(m.weights["router_w"], m.weights["router_bias"], n, topk=c.topk,
                                      routed_scale=c.routed_scale)              # :836-842, the same on every rank
                loc = (ids.to(torch.int32) & 0xFFFF).view(-1) - self.base
                mine = (loc >= 0) & (loc < self.per)
                e = torch.where(mine, loc, torch.full_like(loc, -1))
                y = m.experts_grouped(n, e.contiguous(), self.zero8)             # rows of experts held elsewhere stay unwritten
                part = (torch.where(mine[:, None], y.float(), torch.zeros((), device=y.device)) * wts.view(-1, 1)).sum(0)
                if self.world > 1:
                    dist.all_reduce(part, group=self.group)                      # the layer's only exchange: 4 x hidden bytes
                t = part.bfloat16()                                              # :871
                if c.shared_inter:
                    t = (t.float() + m.shared(n).float().view(-1)).bfloat16()    # :872-875 (:684)
                t = t.view(1, -1)
            last = l + 1 == len(self.layers)
            n = lib.add_rmsnorm(x, t, self.norm if last else self.layers[l + 1]["ln0"],
                                eps=c.final_rms_eps if last else c.rms_eps)      # :877, then :812 / :880
        self.ids_out.copy_(lib.lm_head_argmax(self.lm_head, n).view(-1).to(torch.int32))
        self.pos += 1

    def step(self, ids):
        """ids int32 [1] on the device -> the greedy next id (int32 [1], device)."""
        self.ids_in.copy_(ids.view(-1))
        if self.graph is not None:
            self.graph.replay()
        elif self.use_graph and self.steps >= 1 and torch.cuda.current_stream(self.device) != torch.cuda.default_stream(self.device):
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=torch.cuda.current_stream(self.device)):
                    self._body()
                self.graph = g
                g.replay()
            except Exception:  # capture not possible in this set-up: stay eager (and keep the ranks in step)
                self.use_graph, self.graph = False, None
                torch.cuda.synchronize(self.device)
                self._body()
        else:
            self._body()
        self.steps += 1
        return self.ids_out.clone()

    def reset(self):
        self.pos.zero_()

    def generate(self, prompt, max_new):
        """Greedy generation with host token lists (the executor's contract): prompt replayed token by token."""
        self.reset()
        out, nxt = [], None
        for tok in prompt:
            nxt = self.step(torch.tensor([tok], dtype=torch.int32, device=self.device))
        for _ in range(max_new):
            tok = int(nxt.item())
            if tok == self.cfg.eos_id:
                break
            out.append(tok)
            nxt = self.step(nxt)
        return out


def provider_from_model(model, rank, world, device):
    """Cuts a single-GPU lib.Model's tensors for `rank` (tests: the sharded model must generate the same tokens)."""
    import numpy as np
    c = model.cfg
    per = c.experts // world
    shapes = {"gate_w": (c.experts, c.inter, c.hidden // 8), "up_w": (c.experts, c.inter, c.hidden // 8),
              "down_w": (c.experts, c.hidden, c.inter // 8), "gate_s": (c.experts, c.inter, c.hidden // 32),
              "up_s": (c.experts, c.inter, c.hidden // 32), "down_s": (c.experts, c.hidden, c.inter // 32)}
    two_d = {"embed_tokens": (c.vocab, c.hidden), "lm_head": (c.vocab, c.hidden), "q_a_proj": (c.q_rank, c.hidden),
             "q_b_proj": (c.heads * (c.qk_nope + c.qk_rope), c.q_rank), "kv_a_proj_with_mqa": (c.kv_rank + c.qk_rope, c.hidden),
             "kv_b_proj": (c.heads * (c.qk_nope + c.v_head), c.kv_rank), "o_proj": (c.hidden, c.heads * c.v_head),
             "gate_proj": (c.dense_inter, c.hidden), "up_proj": (c.dense_inter, c.hidden), "down_proj": (c.hidden, c.dense_inter),
             "router": (c.experts, c.hidden), "shared_gate": (c.shared_inter, c.hidden), "shared_up": (c.shared_inter, c.hidden),
             "shared_down": (c.hidden, c.shared_inter)}

    def get(layer, name):
        if name in shapes:
            dt = np.uint32 if name.endswith("_w") else np.uint16
            a = model.tensor(layer, name, dt, shapes[name])[rank * per:(rank + 1) * per]
            t = torch.from_numpy(np.ascontiguousarray(a).view(np.int32 if dt == np.uint32 else np.int16)).to(device)
            return t if dt == np.uint32 else t.view(torch.bfloat16)
        if name == "router_bias":
            return torch.from_numpy(model.tensor(layer, name, np.float32)).to(device)
        a = model.tensor(layer, name, np.uint16, two_d.get(name))
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(device).view(torch.bfloat16)
    return get


def synthetic_provider(cfg, rank, world, device, seed=4):
    """Seeded synthetic weights of the benchmark's distributions: replicated tensors are drawn with the same seed on
    every rank, a rank's expert shard with a seed of its own."""
    c = cfg
    per = c.experts // world

    def get(layer, name):
        g = synth._gen(device, seed * 1000003 + (layer + 1) * 131 + sum(ord(ch) for ch in name))
        H = c.hidden
        if name in ("gate_w", "up_w", "down_w", "gate_s", "up_s", "down_s"):
            ge = synth._gen(device, seed * 1000003 + (layer + 1) * 131 + sum(ord(ch) for ch in name) + 7919 * (rank + 1))
            rows, cols = (H, c.inter) if name.startswith("down") else (c.inter, H)
            if name.endswith("_w"):
                return torch.randint(-2 ** 31, 2 ** 31 - 1, (per, rows, cols // 8), generator=ge, device=device, dtype=torch.int32)
            return (torch.randn((per, rows, cols // 32), generator=ge, device=device) * 0.003).abs().bfloat16()
        if name == "router_bias":
            return torch.randn(c.experts, generator=g, device=device) * 0.01
        if name in ("input_layernorm", "post_attention_layernorm", "norm", "kv_a_layernorm"):
            return torch.ones(c.kv_rank if name == "kv_a_layernorm" else H, dtype=torch.bfloat16, device=device)
        if name == "q_a_layernorm":
            return torch.ones(c.q_rank, dtype=torch.bfloat16, device=device)
        shape = {"embed_tokens": (c.vocab, H), "lm_head": (c.vocab, H), "q_a_proj": (c.q_rank, H),
                 "q_b_proj": (c.heads * (c.qk_nope + c.qk_rope), c.q_rank), "kv_a_proj_with_mqa": (c.kv_rank + c.qk_rope, H),
                 "kv_b_proj": (c.heads * (c.qk_nope + c.v_head), c.kv_rank), "o_proj": (H, c.heads * c.v_head),
                 "gate_proj": (c.dense_inter, H), "up_proj": (c.dense_inter, H), "down_proj": (H, c.dense_inter),
                 "router": (c.experts, H), "shared_gate": (c.shared_inter, H), "shared_up": (c.shared_inter, H),
                 "shared_down": (H, c.shared_inter)}[name]
        return synth.normal_bf16(shape, g, device, 0.006)
    return get


def provider_from_index(index_path, cfg, rank, world, device):
    """Tensors for `rank` read from a materialised checkpoint: the text index "blok-runtime-index-v1" of the
    reference's scripts/model_fetch.py:113-127 is first checked against the forward contract for cfg
    (blok_index_validate: src/kimi_exec.cu:736-778), then every tensor this rank needs is read once from its byte
    range [data, data + data_bytes) of the shard file; a rank reads only the experts it owns (experts / world of
    them, stacked expert-major as the kernels expect)."""
    import numpy as np
    lib.index_validate(index_path, cfg)
    entries = {}
    with open(index_path) as fh:
        fh.readline()
        for line in fh:
            f = line.split()
            # tensor name role layer expert slot dtype shape off bytes align data data_bytes file
            entries[(int(f[3]), int(f[4]), f[2], f[5])] = (f[6], f[7], int(f[11]), int(f[12]), f[13])
    per = cfg.experts // world
    names = {"input_layernorm": ("resident", "input_layernorm"), "post_attention_layernorm": ("resident", "post_attention_layernorm"),
             "embed_tokens": ("resident", "embed_tokens"), "norm": ("resident", "norm"), "lm_head": ("resident", "lm_head"),
             "gate_proj": ("dense_ffn_rowcol", "gate_proj"), "up_proj": ("dense_ffn_rowcol", "up_proj"),
             "down_proj": ("dense_ffn_rowcol", "down_proj"), "router": ("router", "gate"),
             "router_bias": ("router", "e_score_correction_bias"), "shared_gate": ("shared_expert_resident", "gate_proj"),
             "shared_up": ("shared_expert_resident", "up_proj"), "shared_down": ("shared_expert_resident", "down_proj")}
    for n in ("q_a_proj", "q_a_layernorm", "q_b_proj", "kv_a_proj_with_mqa", "kv_a_layernorm", "kv_b_proj", "o_proj"):
        names[n] = ("attention_resident", n)
    experts = {"gate_w": "gate_proj.weight_packed", "gate_s": "gate_proj.weight_scale", "up_w": "up_proj.weight_packed",
               "up_s": "up_proj.weight_scale", "down_w": "down_proj.weight_packed", "down_s": "down_proj.weight_scale"}

    def read(key):
        dtype, shape, data, nbytes, path = entries[key]
        with open(path, "rb") as fh:
            fh.seek(data)
            raw = fh.read(nbytes)
        if len(raw) != nbytes:
            raise lib.BlokError(-1, "short read of %s from %s" % (key, path))
        a = np.frombuffer(raw, dtype=np.int32 if dtype == "i32" else np.int16)
        return a.reshape([int(d) for d in shape.split("x")])

    def get(layer, name):
        if name in experts:
            parts = [read((layer, e, "routed_expert", experts[name])) for e in range(rank * per, (rank + 1) * per)]
            t = torch.from_numpy(np.stack(parts)).to(device)
            return t if name.endswith("_w") else t.view(torch.bfloat16)
        role, slot = names[name]
        t = torch.from_numpy(read((layer, -1, role, slot)).copy()).to(device).view(torch.bfloat16)
        return t.float() if name == "router_bias" else t     # the correction bias is fp32 at the ABI
    return get
