"""Cross-cutting helpers: tracing spans and structured logs."""
from .tracing import Tracer, get_tracer, span, start_inference_span, start_request_span
