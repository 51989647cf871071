"""CPU checkers for the retrieval path.  Test infrastructure: the shipped package never imports this."""
