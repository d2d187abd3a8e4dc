"""Events, math helpers, environment bring-up and timing utilities."""
from .event import EventHandle, EventOverlap

__all__ = ["EventHandle", "EventOverlap"]
