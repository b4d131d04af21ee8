// Unbounded multi-producer / single-consumer queue used between the socket thread and the GPU
// workers (same role as the reference's server/include/mpsc.hpp:13-45; admission limits are
// enforced by the caller, not here).
//
// Intrusive singly linked list with a stub node.  A producer publishes in two steps: swap itself
// in as the new tail, then link the previous tail to it.  Between those steps the consumer may see
// the list end early; try_pop() then reports "empty" and the caller retries after its next wake-up,
// so no element is lost or reordered per producer.  Only the consumer frees nodes, and only a node
// whose successor it has already observed, so no producer can still be touching it.  Destroy only
// after all producers and the consumer have stopped.
#pragma once
#include <atomic>
#include <utility>

namespace tib::server {

template <class T>
class MpscQueue {
 public:
  MpscQueue() : head_(new Node), tail_(head_) {}
  MpscQueue(const MpscQueue&) = delete;
  MpscQueue& operator=(const MpscQueue&) = delete;
  ~MpscQueue() {
    for (Node* n = head_; n;) {
      Node* next = n->next.load(std::memory_order_relaxed);
      delete n;
      n = next;
    }
  }

  void push(T value) {
    Node* node = new Node;
    node->item = std::move(value);
    Node* before = tail_.exchange(node, std::memory_order_acq_rel);
    before->next.store(node, std::memory_order_release);
  }

  // Consumer only.  False when nothing is linked yet.
  bool try_pop(T& out) {
    Node* first = head_->next.load(std::memory_order_acquire);
    if (!first) return false;
    out = std::move(first->item);
    first->item = T();
    delete head_;
    head_ = first;                  // `first` becomes the new stub
    return true;
  }

 private:
  struct Node {
    std::atomic<Node*> next{nullptr};
    T item{};
  };
  Node* head_;                       // consumer side
  alignas(64) std::atomic<Node*> tail_;
};

}  // namespace tib::server
