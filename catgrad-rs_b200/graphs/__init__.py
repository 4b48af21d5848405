"""The op streams the catgrad model graphs send to a `Backend`, replayed call by call.

These modules stand where `Interpreter::run` + catgrad's stdlib + the catgrad-llm model
graphs stand in the reference: each function issues exactly the backend calls, in the
order, that the cited reference function lowers to.  They work on any object with the
trait's methods (catgrad/src/interpreter/backend/mod.rs:22-82), so the same stream drives
the CUDA backend and a checker.
"""
from . import nn, helpers, llama, qwen3, gemma, gpt2, granite, deepseek, llama_kv  # noqa: F401
