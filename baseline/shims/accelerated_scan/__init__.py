"""Import-time stand-in for the `accelerated_scan` package: the first-order linear recurrence restated in PyTorch."""
