"""Analytic performance model (roofline) and report formats."""
from .roofline import DEVICES, DeviceLimits, RooflinePlan, estimate, format_report, report_json

__all__ = ["DEVICES", "DeviceLimits", "RooflinePlan", "estimate", "format_report", "report_json"]
