"""Offline harnesses."""
