#!/usr/bin/env python3
"""Text generation with LLMPipeline on the CUDA device.

usage: llm_generate.py <model dir with openvino_model.xml | model.gguf> "<prompt>" [max_new_tokens]
Without a tokenizer file next to the model the byte-level tokenizer is used.
"""
import sys

from openvino_b200.genai import GenerationConfig, LLMPipeline


def main() -> int:
    if len(sys.argv) < 3:
        print(__doc__)
        return 1
    pipe = LLMPipeline(sys.argv[1], "CUDA")
    cfg = GenerationConfig(max_new_tokens=int(sys.argv[3]) if len(sys.argv) > 3 else 64)
    print(pipe.generate(sys.argv[2], cfg))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
