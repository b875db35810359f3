"""CUDA-graph decode wrapper: mirror of inference/graph_wrapper.py:21-212 (GLoRCQGraphWrapper) and
218-290 (run_speed_benchmark).

Prefill runs eagerly with a dynamic length; one decode step (batch x 1 token) is captured once and
replayed per token from static buffers: ``static_input_ids (B,1) int64``, ``static_cache_position (1,)
int64``, ``static_logits (B,1,V)``, and a static key/value cache.  The MoE blocks need no mode switch
here (one device-side path serves eager and captured execution); ``graph_mode`` is still toggled for
hosts that read it.
"""

from __future__ import annotations

import gc
import time

import torch

from .decoder import StaticKVCache as StaticCache
from .moe_block import GraphCompatibleMoeBlock
from .parallel import PeerExchange


class GLoRCQGraphWrapper:
    """wrapper = GLoRCQGraphWrapper(model, max_batch_size=1, max_seq_len=4096)
    output_ids, seconds = wrapper.generate(input_ids, max_new_tokens=128)"""

    def __init__(self, model, max_batch_size=1, max_seq_len=4096):
        self.model = model
        self.max_batch_size = max_batch_size
        self.max_seq_len = max_seq_len
        self.device = next(model.parameters()).device
        self.dtype = next(model.parameters()).dtype
        self.static_cache = StaticCache(config=model.config, max_batch_size=max_batch_size, max_cache_len=max_seq_len,
                                        device=self.device, dtype=self.dtype)
        self.static_input_ids = torch.zeros((max_batch_size, 1), dtype=torch.long, device=self.device)
        self.static_cache_position = torch.zeros((1,), dtype=torch.long, device=self.device)
        self.static_logits = None
        self.static_next = None
        # this package's decoder can skip the logits of all prompt positions but the last
        import inspect
        self._keep_last_only = "logits_to_keep" in inspect.signature(model.forward).parameters
        self.graph = None
        self.graph_stream = torch.cuda.Stream(device=self.device)
        self.last_prefill_seconds = None
        self.last_decode_seconds = None

    def _set_moe_graph_mode(self, mode: bool):
        for module in self.model.modules():
            if isinstance(module, GraphCompatibleMoeBlock):
                module.graph_mode = mode

    def _step(self):
        return self.model(input_ids=self.static_input_ids, cache_position=self.static_cache_position,
                          past_key_values=self.static_cache, use_cache=True, return_dict=False)

    def capture_graph(self):
        """Allocation pass, three warm-up steps on a side stream, then the recorded step
        (inference/graph_wrapper.py:69-130)."""
        self.model.eval()
        self._set_moe_graph_mode(True)
        with torch.no_grad():
            self.static_input_ids.fill_(1)
            self.static_cache_position.fill_(0)
            self._step()
        torch.cuda.synchronize()
        gc.collect()
        torch.cuda.empty_cache()
        # (warm-up on the stream the capture will use: per-stream workspaces are then found, not made, while capturing)
        s = self.graph_stream
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(3):
                self.static_input_ids.fill_(1)
                self.static_cache_position.fill_(10 if self.max_seq_len > 10 else 0)
                self._step()
        torch.cuda.current_stream().wait_stream(s)
        gc.collect()
        torch.cuda.empty_cache()
        self.graph = torch.cuda.CUDAGraph()
        self.static_input_ids.fill_(1)
        self.static_cache_position.fill_(0)
        with torch.cuda.graph(self.graph, stream=self.graph_stream), torch.no_grad():
            self.static_logits = self._step()[0]
        # the model's output projection may leave the greedy token of the step beside the logits
        best = getattr(self.model, "last_argmax", None)
        self.static_next = best.view(self.max_batch_size, 1) if best is not None else None

    @torch.no_grad()
    def replay(self, input_ids, cache_position_val):
        assert input_ids.shape[0] == self.max_batch_size, \
            f"Input batch size {input_ids.shape[0]} != graph batch size {self.max_batch_size}"
        self.static_input_ids.copy_(input_ids)
        self.static_cache_position.fill_(cache_position_val)
        self.graph.replay()
        return self.static_logits

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=100):
        """Greedy decoding: eager prefill, graph replay per new token.  Returns (ids (B, T + new),
        seconds) like the reference (inference/graph_wrapper.py:152-212)."""
        start = time.time()
        batch_size, seq_len = input_ids.shape
        assert batch_size == self.max_batch_size, \
            f"Input batch_size ({batch_size}) must match max_batch_size ({self.max_batch_size})"
        output_ids = input_ids.clone()
        self._set_moe_graph_mode(False)
        self.static_cache.reset()
        kw = {"logits_to_keep": 1} if self._keep_last_only else {}
        logits = self.model(input_ids=input_ids, cache_position=torch.arange(seq_len, device=self.device),
                            past_key_values=self.static_cache, use_cache=True, return_dict=False, **kw)[0]
        next_token = torch.argmax(logits[:, -1, :], dim=-1, keepdim=True)
        output_ids = torch.cat([output_ids, next_token], dim=1)
        torch.cuda.synchronize()
        prefill_end = time.time()
        self._set_moe_graph_mode(True)
        if self.graph is None:
            # capturing runs steps at positions 0 and 10 of the static cache: keep the prompt's entries
            keep_k, keep_v = self.static_cache.k[:, :, :, :11].clone(), self.static_cache.v[:, :, :, :11].clone()
            self.capture_graph()
            self.static_cache.k[:, :, :, :11].copy_(keep_k)
            self.static_cache.v[:, :, :, :11].copy_(keep_v)
            torch.cuda.synchronize()
            prefill_end = time.time()
        for i in range(max_new_tokens - 1):
            pos = seq_len + i
            if pos >= self.max_seq_len:
                break
            logits = self.replay(next_token, pos)
            if self.static_next is not None:
                next_token = self.static_next.clone()         # arg-max taken inside the captured step
            else:
                next_token = torch.argmax(logits[:, -1, :], dim=-1, keepdim=True)
            output_ids = torch.cat([output_ids, next_token], dim=1)
        torch.cuda.synchronize()
        end = time.time()
        PeerExchange.check_all()      # expert parallel: a wait for another rank that ran out invalidates the tokens
        self.last_prefill_seconds, self.last_decode_seconds = prefill_end - start, end - prefill_end
        return output_ids, end - start


def run_speed_benchmark(model, tokenizer=None, max_batch_size=1, max_seq_len=2048, prompt_len=128, gen_len=128,
                        input_ids=None):
    """Eager greedy generation against graph replay (inference/graph_wrapper.py:218-290).  The prompt is
    `input_ids` when given, else `prompt_len` random characters through `tokenizer` as in the reference."""
    device = next(model.parameters()).device
    if input_ids is None:
        import random
        import string
        alphabet = string.ascii_letters + string.digits + " "
        prompt = "".join(random.choice(alphabet) for _ in range(prompt_len))
        input_ids = tokenizer(prompt, return_tensors="pt", max_length=prompt_len, truncation=True).input_ids
    input_ids = input_ids.to(device)
    torch.cuda.synchronize()
    t0 = time.time()
    with torch.no_grad():
        model.generate(input_ids, max_new_tokens=gen_len, do_sample=False)
    torch.cuda.synchronize()
    t_std = time.time() - t0
    wrapper = GLoRCQGraphWrapper(model, max_batch_size=max_batch_size, max_seq_len=max_seq_len)
    wrapper.capture_graph()
    torch.cuda.synchronize()
    _, t_graph = wrapper.generate(input_ids, max_new_tokens=gen_len)
    std_tps, graph_tps = gen_len / t_std, gen_len / t_graph
    return {"standard_tps": std_tps, "graph_tps": graph_tps, "speedup": graph_tps / std_tps if std_tps > 0 else 0}
