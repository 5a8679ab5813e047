"""CPU checker for the KVComp hot path.  Test infrastructure: the product never imports it."""
