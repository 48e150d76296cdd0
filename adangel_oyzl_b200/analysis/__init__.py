from .report import generate_report

__all__ = ["generate_report"]
