"""Serving front ends: OpenAI-compatible HTTP server, chat templating, tool-call and reasoning
parsers, the asynchronous engine wrapper and the command-line tools."""
