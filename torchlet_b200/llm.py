"""Python entry point and command line, in the reference's manner.

The reference: ``LLM(model_id, max_decode_slots=4, kv_block_size=16,
max_num_blocks=None)`` and ``await llm.generate(list[str], max_new_tokens=128) ->
list[str]`` (v10_triton_paged_gqa/llm.py:20-110), run as
``python -m torchlet.v10_triton_paged_gqa.llm`` with three built-in prompts
(llm.py:113-140).  Same names and meanings here: ``max_decode_slots`` is the most
requests live at a time, ``kv_block_size`` the tokens per cache page, ``max_num_blocks``
the size of the page pool including the reserved page 0.  Differences: the model comes
from a local folder, prompts may also be lists of token ids (returned as token ids), and
sampling options can be given.  ``generate`` is synchronous; ``agenerate`` is the reference's
coroutine: several may run at once, each handing its requests to the one engine loop, which is
an asyncio task until ``await llm.shutdown()``.  Run without prompts, the command line does what
the reference's does: three ``agenerate`` tasks that start a tenth of a second apart.

    python -m torchlet_b200.llm --model DIR --prompt "hello" --max-new-tokens 64
    python -m torchlet_b200.llm --model DIR --prompt-ids 1,2,3 --temperature 0.8 --seed 7
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Optional, Sequence, Union

from .config import EngineConfig
from .logger import logger
from .sampling import SamplingParams


def _load_tokenizer(model_dir: Path):
    """The folder's tokenizer, if it has one (transformers' AutoTokenizer, as the reference)."""
    if not any((model_dir / name).is_file() for name in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
        return None
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(str(model_dir))


class LLM:
    def __init__(self, model_dir: Union[str, Path], max_decode_slots: int = 4, kv_block_size: int = 16,
                 max_num_blocks: Optional[int] = None, dtype: str = "bfloat16",
                 max_seq_len: Optional[int] = None, max_num_batched_tokens: int = 2048,
                 cuda_graph: bool = True, device: str = "cuda:0", admission_headroom: Optional[int] = 1):
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is required")
        from .engine.engine import Engine
        from .engine.loading import load_model

        from .utils import get_backend_info

        logger.info("backend info:\n%s", get_backend_info())
        self.model_dir = Path(model_dir)
        self.engine_config = EngineConfig(
            dtype=dtype, max_decode_slots=max_decode_slots, kv_block_size=kv_block_size,
            max_num_blocks=max_num_blocks, max_seq_len=max_seq_len,
            max_num_batched_tokens=max_num_batched_tokens, cuda_graph=cuda_graph, device=device,
            admission_headroom=admission_headroom)
        self.model = load_model(self.model_dir, self.engine_config.dtype, device)
        self.config = self.model.config
        self.tokenizer = _load_tokenizer(self.model_dir)
        self.stop_ids = set()
        if self.tokenizer is not None:
            candidates = {self.tokenizer.eos_token_id, self.tokenizer.convert_tokens_to_ids("<|im_end|>")}
            self.stop_ids = {t for t in candidates if isinstance(t, int) and t >= 0}
        elif getattr(self.config, "eos_token_id", None) is not None:
            self.stop_ids = {int(self.config.eos_token_id)}
        self.engine = Engine(self.model, self.engine_config)
        logger.info("engine ready: %s", self.engine_config)

    @classmethod
    def from_model(cls, model, max_decode_slots: int = 4, kv_block_size: int = 16,
                   max_num_blocks: Optional[int] = None, max_seq_len: Optional[int] = None,
                   max_num_batched_tokens: int = 2048, cuda_graph: bool = True, device: str = "cuda:0") -> "LLM":
        """An ``LLM`` around a model that is already on the device (no folder, no tokenizer)."""
        from .engine.engine import Engine

        self = cls.__new__(cls)
        dtype = "bfloat16" if str(model.dtype).endswith("bfloat16") else "float32"
        self.model_dir, self.model, self.config = None, model, getattr(model, "config", None)
        self.engine_config = EngineConfig(
            dtype=dtype, max_decode_slots=max_decode_slots, kv_block_size=kv_block_size,
            max_num_blocks=max_num_blocks, max_seq_len=max_seq_len,
            max_num_batched_tokens=max_num_batched_tokens, cuda_graph=cuda_graph, device=device)
        self.tokenizer, self.stop_ids = None, set()
        self.engine = Engine(self.model, self.engine_config)
        return self

    def _encode(self, prompts: Sequence[str]) -> list:
        if self.tokenizer is None:
            raise ValueError("text prompts need tokenizer files in the model folder; pass token ids instead")
        texts = prompts
        if getattr(self.tokenizer, "chat_template", None):
            texts = [
                self.tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False,
                                                   add_generation_prompt=True)
                for p in prompts
            ]
        return self.tokenizer(list(texts), padding=False)["input_ids"]

    def _requests(self, inputs: Sequence, max_new_tokens: int, sampling_params) -> list:
        from .engine.scheduler import Request

        as_text = isinstance(inputs[0], str)
        token_lists = self._encode(inputs) if as_text else [list(i) for i in inputs]
        requests = []
        for i, tokens in enumerate(token_lists):
            if sampling_params is None:
                params = SamplingParams(max_new_tokens=max_new_tokens)
            elif isinstance(sampling_params, SamplingParams):
                params = SamplingParams(**vars(sampling_params))
            else:
                params = SamplingParams(**vars(sampling_params[i]))
            if not params.stop_token_ids and not params.ignore_eos:
                params.stop_token_ids = tuple(sorted(self.stop_ids))
            requests.append(Request(tokens, params, prompt=inputs[i] if as_text else ""))
        return requests

    def _outputs(self, requests: list, as_text: bool) -> list:
        for request in requests:
            if request.error is not None:
                raise request.error
        if as_text:
            outputs = self.tokenizer.batch_decode([r.output_tokens for r in requests], skip_special_tokens=True)
            for request, text in zip(requests, outputs):
                request.output = text
            return list(outputs)
        return [list(r.output_tokens) for r in requests]

    def generate(self, inputs: Sequence, max_new_tokens: int = 128,
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> list:
        """Generate for every input.  Text inputs give text outputs, token-id inputs give
        lists of token ids.  ``sampling_params`` (one for all, or one per input)
        overrides ``max_new_tokens``."""
        if not inputs:
            return []
        if max_new_tokens <= 0 and sampling_params is None:
            return ["" if isinstance(i, str) else [] for i in inputs]
        requests = self._requests(inputs, max_new_tokens, sampling_params)
        self.engine.generate(requests)
        return self._outputs(requests, isinstance(inputs[0], str))

    async def agenerate(self, inputs: Sequence, max_new_tokens: int = 128,
                        sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> list:
        """``generate`` as a coroutine, the reference's form (llm.py:84-110): the requests join the
        engine loop, which runs as an asyncio task and batches them with those of every other
        ``agenerate`` that is waiting; returns when these have ended.  Not to be mixed with a
        synchronous ``generate`` while the task lives (``await llm.shutdown()`` ends it)."""
        if not inputs:
            return []
        if max_new_tokens <= 0 and sampling_params is None:
            return ["" if isinstance(i, str) else [] for i in inputs]
        requests = self._requests(inputs, max_new_tokens, sampling_params)
        await self.engine.submit(requests)
        return self._outputs(requests, isinstance(inputs[0], str))

    async def shutdown(self) -> None:
        """Ends the engine loop's task; requests still live end with ``asyncio.CancelledError``."""
        await self.engine.shutdown()


def _three_arrivals(llm: "LLM", params: SamplingParams) -> int:
    """The reference's own demonstration (llm.py:113-140): its three built-in prompts as three
    coroutines that start a tenth of a second apart, served by one engine loop."""
    import asyncio

    prompts = ["hello, do a simple introduction", "what's the nearest star", "write a short haiku about GPUs"]

    async def arrive() -> list:
        try:
            tasks = []
            for prompt in prompts:
                tasks.append(asyncio.create_task(llm.agenerate([prompt], sampling_params=params)))
                await asyncio.sleep(0.1)
            return await asyncio.gather(*tasks)
        finally:
            await llm.shutdown()

    for i, outputs in enumerate(asyncio.run(arrive()), start=1):
        print(f"batch {i}:")
        print(outputs)
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m torchlet_b200.llm", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    parser.add_argument("--prompt", action="append", default=[], help="text prompt (needs tokenizer files); repeatable")
    parser.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeatable")
    parser.add_argument("--max-new-tokens", type=int, default=64)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=None)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--max-decode-slots", type=int, default=4)
    parser.add_argument("--kv-block-size", type=int, default=16)
    parser.add_argument("--max-num-blocks", type=int, default=None)
    parser.add_argument("--max-seq-len", type=int, default=None)
    parser.add_argument("--max-num-batched-tokens", type=int, default=2048)
    parser.add_argument("--no-cuda-graph", action="store_true")
    parser.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                        help="first write random weights (this seed) into --model, which must hold a config.json")
    args = parser.parse_args(argv)

    if args.random_weights is not None:
        from .config import load_config
        from .weights import write_random_model

        write_random_model(args.model, load_config(args.model), args.random_weights)
    llm = LLM(args.model, max_decode_slots=args.max_decode_slots, kv_block_size=args.kv_block_size,
              max_num_blocks=args.max_num_blocks, dtype=args.dtype, max_seq_len=args.max_seq_len,
              max_num_batched_tokens=args.max_num_batched_tokens, cuda_graph=not args.no_cuda_graph)
    params = SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature, seed=args.seed,
                            ignore_eos=args.ignore_eos)
    if args.prompt_ids:
        prompts = [[int(t) for t in item.split(",") if t.strip()] for item in args.prompt_ids]
    elif args.prompt:
        prompts = args.prompt
    else:
        return _three_arrivals(llm, params)
    outputs = llm.generate(prompts, sampling_params=params)
    for i, output in enumerate(outputs, start=1):
        print(f"output {i}:")
        print(output if isinstance(output, str) else json.dumps(output))
    return 0


if __name__ == "__main__":
    sys.exit(main())
